// Grouped-query attention over a paged K/V pool for ragged batches, with the pieces a parallel-sublayer
// decoder adds to it:
//   rope_append_kernel   rotary positions on the first rot_dims columns of every q / k head (pairs
//                        (2i, 2i+1) or (i, i + rot_dims / 2), angle = position * inv_freq[i], evaluated in
//                        double so that far positions keep their phase; cos and sin optionally scaled by
//                        one magnitude), optional unit norm per head (fp32), q out as fp32,
//                        k | v appended to the pool row of the token
//   paged_attn_kernel    fp32 scores of ALL H heads of a (query, key) pair, optional head mixing
//                        s_h <- sum_g talk[h, g] s_g before the softmax, online softmax whose running
//                        (max, sum) starts at (sink_h, 1) when a sink is given, fp32 weighted sum.
//                        A CTA owns BQ consecutive rows of one sequence x all heads (BQ * H "score rows");
//                        prompt portions use BQ up to 16, decoded tokens BQ = 1 with the key blocks of a
//                        row dealt to nsplit CTAs
//   paged_attn_merge_kernel  merges the nsplit partial (max, sum, weighted sum) triples of a decoded token
// Options another architecture can combine freely: an additive bias looked up by the distance between
// query and key (dist_bias [dist_rows, H], the last row serves every larger distance; added after scale and
// mixing), a chunked mask (a query sees the keys of its own block of `chunk` positions only; the key loop
// starts at the block of the tile's first row), and a per-(token, head) sigmoid gate on the output.
// A sliding window with kept first tokens (a key is seen if it is at most window - 1 positions back, or among the
// first keep_first of its sequence) is a mask plus a shorter block list: the blocks that hold kept tokens, then
// the blocks from the window of the tile's first row on.  A per-head multiplier of the scores is folded into the
// staged queries.  talk_after mixes the heads' softmax WEIGHTS: that needs every head's final (max, sum) before
// any value is added, so the kernels first run over the key blocks with the scores only (pass 0), then again with
// weights exp(s - max) / sum, mixed over heads, times the values (pass 1; nothing is rescaled).  When the keys of
// a decoded token are dealt to several CTAs, pass 0 and pass 1 are two launches: the first leaves every CTA's
// (max, sum) of its share in the partial records, the second merges them in split order and adds its share.
// Every reduction over keys runs in key order inside a block and block by block, so a row's result does
// not depend on what else is in the launch.
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr float kNegBig = -1e30f;

__host__ __device__ __forceinline__ int round4(int r) { return (r + 3) & ~3; }
// Floats between the K rows of consecutive keys in shared memory: all G heads of a key (G * DS, DS = D4 + 4)
// plus a pad that makes the stride 4 mod 32, so that the float4 reads of 8 consecutive keys (same head, same
// column) fall into 8 different bank groups.
__host__ __device__ __forceinline__ int key_stride(int G, int DS) { return G * DS + ((36 - (G * DS) % 32) % 32); }

// ---- rotary + unit norm + append ---------------------------------------------------------------------
// One CTA per token; warp w takes the heads w, w + 8, ... of q then k; v is copied by all threads.
__global__ void __launch_bounds__(kThreads) rope_append_kernel(const vila_rope_append_params p) {
  extern __shared__ float cs[];   // cos [rot/2] | sin [rot/2]
  const int t = blockIdx.x, half = p.rot_dims >> 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const double pos = static_cast<double>(p.positions[t]);
  const float mag = p.rot_mscale != 0.f ? p.rot_mscale : 1.0f;
  for (int i = tid; i < half; i += kThreads) {
    double s, c;
    sincos(pos * p.inv_freq[i], &s, &c);
    cs[i] = static_cast<float>(c) * mag;
    cs[half + i] = static_cast<float>(s) * mag;
  }
  __syncthreads();
  // column c of the rotated part: its partner, its pair index and whether it is the second of its pair
  const bool halves = p.rot_layout == 1;
  auto partner = [&](int c) { return halves ? (c < half ? c + half : c - half) : (c ^ 1); };
  auto pair_of = [&](int c) { return halves ? (c < half ? c : c - half) : (c >> 1); };
  auto second = [&](int c) { return halves ? c >= half : (c & 1) != 0; };
  const size_t in0 = static_cast<size_t>(t) * p.ldq;
  const size_t prow = static_cast<size_t>(p.cache_rows[t]) * (static_cast<size_t>(p.G) * (p.dim + p.vdim));
  for (int hh = warp; hh < p.H + p.G; hh += kWarps) {
    const bool is_q = hh < p.H;
    const size_t src = in0 + static_cast<size_t>(hh) * p.dim;   // q heads then k heads are contiguous
    // pass 1: rotated values -> sum of squares (recomputed in pass 2: dim is small, no buffer needed)
    float ss = 0.f;
    for (int c = lane; c < p.dim; c += 32) {
      float v = ld_any(p.qkv, p.qkv_dtype, src + c);
      if (c < p.rot_dims) {
        const float o = ld_any(p.qkv, p.qkv_dtype, src + partner(c));
        const float co = cs[pair_of(c)], si = cs[half + pair_of(c)];
        v = second(c) ? fmaf(v, co, o * si) : fmaf(v, co, -(o * si));
      }
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = p.unit_norm ? 1.0f / sqrtf(ss / static_cast<float>(p.dim) + p.eps) : 1.0f;
    const float* nw = is_q ? p.q_norm_w : p.k_norm_w;
    for (int c = lane; c < p.dim; c += 32) {
      float v = ld_any(p.qkv, p.qkv_dtype, src + c);
      if (p.v_from_k && !is_q)   // the value is the key as it came in
        st_any(p.pool, p.pool_dtype, prow + static_cast<size_t>(p.G) * p.dim + static_cast<size_t>(hh - p.H) * p.dim + c, v);
      if (c < p.rot_dims) {
        const float o = ld_any(p.qkv, p.qkv_dtype, src + partner(c));
        const float co = cs[pair_of(c)], si = cs[half + pair_of(c)];
        v = second(c) ? fmaf(v, co, o * si) : fmaf(v, co, -(o * si));
      }
      v *= r;
      if (nw) v *= nw[c];
      if (is_q) p.q_out[(static_cast<size_t>(t) * p.H + hh) * p.dim + c] = v;
      else st_any(p.pool, p.pool_dtype, prow + static_cast<size_t>(hh - p.H) * p.dim + c, v);
    }
  }
  if (p.v_from_k) return;
  const size_t vsrc = in0 + static_cast<size_t>(p.H + p.G) * p.dim, vdst = prow + static_cast<size_t>(p.G) * p.dim;
  for (int c = tid; c < p.G * p.vdim; c += kThreads)
    st_any(p.pool, p.pool_dtype, vdst + c, ld_any(p.qkv, p.qkv_dtype, vsrc + c));
}

// ---- attention -----------------------------------------------------------------------------------------
struct AttnShape {
  int BQ;      // query rows per CTA
  int BK;      // keys per block (<= 32: one lane per key in the softmax step)
  int sub;     // CTAs per 16-row tile (grid.y)
  int hsplit;  // head groups per tile (grid.z of the tiled kernel): 1 = all heads in one CTA, G = one K/V head and
               // its query heads per CTA (possible when the heads' scores are not mixed)
  int phase;   // weights mixed after the softmax with the keys of a row dealt to several CTAs: 0 = this launch only
               // leaves every CTA's running (max, sum) in its partial record, 1 = this launch merges those records and
               // adds its share of the values; -1 = one CTA does both passes itself
};

__device__ __forceinline__ size_t pool_row(const int32_t* pt, int page, int j) {
  return static_cast<size_t>(pt[j / page]) * page + (j % page);
}

// first key a query at position pos can see
__device__ __forceinline__ int first_key(const vila_paged_attn_params& p, int pos) {
  return p.chunk > 0 ? (pos / p.chunk) * p.chunk : 0;
}
// may the query at position pos see key j?
__device__ __forceinline__ bool sees(const vila_paged_attn_params& p, int pos, int j) {
  return j <= pos && j >= first_key(p, pos) && (p.window <= 0 || pos - j < p.window || j < p.keep_first);
}
// Key blocks of BK keys a tile visits, in order: [0, kb) then [wb, nblocks).
struct BlockList {
  int kb, wb, count;
  __device__ __forceinline__ int block(int v) const { return v < kb ? v : wb + (v - kb); }
};
__device__ __forceinline__ BlockList visible_blocks(const vila_paged_attn_params& p, int pos0, int nkeys, int BK) {
  BlockList b;
  const int nblocks = (nkeys + BK - 1) / BK;
  if (p.window <= 0) {
    b.kb = 0;
    b.wb = first_key(p, pos0) / BK;
  } else {
    b.kb = min((min(p.keep_first, nkeys) + BK - 1) / BK, nblocks);
    b.wb = max(b.kb, max(max(pos0 - p.window + 1, 0), first_key(p, pos0)) / BK);
  }
  b.count = b.kb + max(nblocks - b.wb, 0);
  return b;
}
__device__ __forceinline__ float head_scale(const vila_paged_attn_params& p, int h) {
  return p.head_scale ? p.scale * p.head_scale[h] : p.scale;
}
__device__ __forceinline__ float dist_bias(const vila_paged_attn_params& p, int dist, int h) {
  return __ldg(p.dist_bias + static_cast<size_t>(min(dist, p.dist_rows - 1)) * p.H + h);
}
__device__ __forceinline__ float out_gate(const vila_paged_attn_params& p, int row, int h) {
  return p.gate ? sigmoid_f(ld_any(p.gate, p.gate_dtype, static_cast<size_t>(row) * p.ldg + h)) : 1.0f;
}

// K | V rows of a key block, widened to fp32: one warp per key.  16-byte loads when the head sizes allow
// (bf16: multiples of 8, fp32: multiples of 4; the pool row is then 16-byte aligned as well).
// g0, G: the K/V heads g0 .. g0 + G - 1 of the pool row are loaded (all of them by default).
__device__ __forceinline__ void load_kv_block(float* Ks, float* Vs, const vila_paged_attn_params& p,
                                              const int32_t* pt, int j0, int nkeys, int BK, int D4, int DS, int V4,
                                              int nwarps = kWarps, int g0 = 0, int G = 0, bool with_v = true) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (G == 0) G = p.G;
  const int D = p.dim, V = p.vdim, KS = key_stride(G, DS);
  const size_t prw = static_cast<size_t>(p.G) * (D + V);
  const size_t koff = static_cast<size_t>(g0) * D, voff = static_cast<size_t>(p.G) * D + static_cast<size_t>(g0) * V;
  const bool vec16 = p.pool_dtype == VILA_DT_BF16 && (D & 7) == 0 && (V & 7) == 0;
  const bool vec32 = p.pool_dtype == VILA_DT_F32 && (D & 3) == 0 && (V & 3) == 0;
  for (int jj = warp; jj < BK; jj += nwarps) {
    const int j = j0 + jj;
    float* kd = Ks + jj * KS;
    float* vd = Vs + jj * G * V4;
    if (j >= nkeys) {
      for (int x = lane; x < KS; x += 32) kd[x] = 0.f;
      for (int x = lane; x < G * V4; x += 32) vd[x] = 0.f;
      continue;
    }
    const size_t src = pool_row(pt, p.page, j) * prw;
    if (vec16) {
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(p.pool) + src;
      const uint4* k4 = reinterpret_cast<const uint4*>(base + koff);
      const uint4* v4 = reinterpret_cast<const uint4*>(base + voff);
      for (int x = lane; x < (G * D) >> 3; x += 32) {
        const uint4 u = __ldg(k4 + x);
        const int e = x << 3, g = e / D, k = e - g * D;
        float* d = kd + g * DS + k;
        *reinterpret_cast<float4*>(d) = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                                                    __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
        *reinterpret_cast<float4*>(d + 4) = make_float4(__uint_as_float(u.z << 16), __uint_as_float(u.z & 0xffff0000u),
                                                        __uint_as_float(u.w << 16), __uint_as_float(u.w & 0xffff0000u));
      }
      for (int x = lane; with_v && x < (G * V) >> 3; x += 32) {
        const uint4 u = __ldg(v4 + x);
        float* d = vd + (x << 3);
        *reinterpret_cast<float4*>(d) = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                                                    __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
        *reinterpret_cast<float4*>(d + 4) = make_float4(__uint_as_float(u.z << 16), __uint_as_float(u.z & 0xffff0000u),
                                                        __uint_as_float(u.w << 16), __uint_as_float(u.w & 0xffff0000u));
      }
    } else if (vec32) {
      const float* base = static_cast<const float*>(p.pool) + src;
      const float4* k4 = reinterpret_cast<const float4*>(base + koff);
      const float4* v4 = reinterpret_cast<const float4*>(base + voff);
      for (int x = lane; x < (G * D) >> 2; x += 32) {
        const int e = x << 2, g = e / D, k = e - g * D;
        *reinterpret_cast<float4*>(kd + g * DS + k) = __ldg(k4 + x);
      }
      for (int x = lane; with_v && x < (G * V) >> 2; x += 32) *reinterpret_cast<float4*>(vd + (x << 2)) = __ldg(v4 + x);
    } else {
      for (int x = lane; x < G * D4; x += 32) {
        const int g = x / D4, k = x - g * D4;
        kd[g * DS + k] = k < D ? ld_any(p.pool, p.pool_dtype, src + koff + static_cast<size_t>(g) * D + k) : 0.f;
      }
      const size_t vsrc = src + voff;
      for (int x = lane; with_v && x < G * V4; x += 32) {
        const int g = x / V4, k = x - g * V4;
        vd[x] = k < V ? ld_any(p.pool, p.pool_dtype, vsrc + static_cast<size_t>(g) * V + k) : 0.f;
      }
    }
  }
}

// Shared memory (floats):  Qs [BQ * H][D4] (scale folded in) | Ks [BK][G][DS] | Vs [BK][G][V4] |
//   Ss [BQ * H][BK] raw scores | Ps [BQ * H][BK] weights | talk [H * H] | m, l, alpha [BQ * H]
// DS = D4 + 4: consecutive keys start 4 banks apart, so the float4 reads of 8 keys do not collide.
template <int NACC>
__global__ void __launch_bounds__(kThreads) paged_attn_kernel(const vila_paged_attn_params p, const AttnShape sh) {
  extern __shared__ __align__(16) float sm[];
  const int H = p.H, G = p.G, D = p.dim, V = p.vdim, BQ = sh.BQ, BK = sh.BK;
  const int D4 = round4(D), DS = D4 + 4, V4 = round4(V), R = BQ * H, rep = H / G, KS = key_stride(G, DS);
  float* Qs = sm;
  float* Ks = Qs + R * D4;
  float* Vs = Ks + BK * KS;
  float* Ss = Vs + BK * G * V4;
  float* Ps = Ss + R * BK;
  float* Tk = Ps + R * BK;
  float* m_s = Tk + H * H;
  float* l_s = m_s + R;
  float* a_s = l_s + R;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int i0 = blockIdx.y * BQ;
  const int n_tile = tile[1];
  if (i0 >= n_tile) return;
  const int row0 = tile[0] + i0, n = min(BQ, n_tile - i0), pos0 = tile[2] + i0;
  const int32_t* pt = p.page_tables + static_cast<size_t>(tile[3]) * p.pt_stride;
  const int split = blockIdx.z, nsplit = gridDim.z;
  const size_t prw = static_cast<size_t>(G) * (D + V);   // pool row width

  for (int idx = tid; idx < R * D4; idx += kThreads) {
    const int r = idx / D4, k = idx - r * D4, i = r / H, h = r - i * H;
    Qs[idx] = (i < n && k < D) ? p.q[(static_cast<size_t>(row0 + i) * H + h) * D + k] * head_scale(p, h) : 0.f;
  }
  for (int idx = tid; idx < H * H; idx += kThreads) Tk[idx] = p.talk ? p.talk[idx] : ((idx / H) == (idx % H) ? 1.f : 0.f);
  const bool after = p.talk_after != 0 && p.talk != nullptr;
  for (int r = tid; r < R; r += kThreads) {
    const bool first = split == 0 && p.sink != nullptr && !after;
    m_s[r] = first ? p.sink[r % H] : kNegBig;
    l_s[r] = first ? 1.0f : 0.0f;
  }
  float4 acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int vq = V4 >> 2;                 // float4 columns of a head
  const int nout = R * vq;                // float4 accumulators of the CTA: index o -> (r, c4)
  const int nkeys = pos0 + n;             // keys 0 .. nkeys - 1 are visible to the last row
  const BlockList bl = visible_blocks(p, pos0, nkeys, BK);

  const int pass_begin = after && sh.phase != 1 ? 0 : 1, pass_end = after && sh.phase == 0 ? 1 : 2;
  for (int pass = pass_begin; pass < pass_end; ++pass) {
  const bool stats = pass == 0;   // scores only: every head's running max and sum over the visible keys
  if (after && !stats) {
    __syncthreads();
    for (int r = tid; r < R; r += kThreads) {
      if (sh.phase == 1) {   // (max, sum) of every split's share, merged in split order
        const int i = r / H, h = r - i * H;
        float mx = kNegBig, l = 0.f;
        if (i < n) {
          const float* rec = p.partial + (static_cast<size_t>(row0 + i) * nsplit * H + h) * (V + 2) + V;
          const size_t step = static_cast<size_t>(H) * (V + 2);
          for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, rec[s * step]);
          for (int s = 0; s < nsplit; ++s) l += expf(rec[s * step] - mx) * rec[s * step + 1];
        }
        m_s[r] = mx;
        l_s[r] = l;
      }
      l_s[r] = l_s[r] > 0.f ? 1.0f / l_s[r] : 0.f;
    }
  }
  const bool all_blocks = stats && sh.phase < 0;
  for (int vb_ = all_blocks ? 0 : split; vb_ < bl.count; vb_ += all_blocks ? 1 : nsplit) {
    const int j0 = bl.block(vb_) * BK;
    __syncthreads();
    load_kv_block(Ks, Vs, p, pt, j0, nkeys, BK, D4, DS, V4, kWarps, 0, 0, !stats);
    __syncthreads();
    // raw scores of every (score row, key)
    for (int idx = tid; idx < R * BK; idx += kThreads) {
      const int r = idx / BK, jj = idx - r * BK, h = r % H;
      const float4* qr = reinterpret_cast<const float4*>(Qs + r * D4);
      const float4* kr = reinterpret_cast<const float4*>(Ks + jj * KS + (h / rep) * DS);
      float s = 0.f;
#pragma unroll 4
      for (int k = 0; k < (D4 >> 2); ++k) {
        const float4 a = qr[k], c = kr[k];
        s = fmaf(a.x, c.x, s); s = fmaf(a.y, c.y, s); s = fmaf(a.z, c.z, s); s = fmaf(a.w, c.w, s);
      }
      Ss[idx] = s;
    }
    __syncthreads();
    if (after) {
      if (stats) {
        // every head's own scores: running max and sum, nothing else
        for (int r = warp; r < R; r += kWarps) {
          const int i = r / H;
          const bool valid = lane < BK && i < n && sees(p, pos0 + i, j0 + lane);
          const float s = valid ? Ss[r * BK + lane] : kNegBig;
          const float m_old = m_s[r];
          const float m_new = fmaxf(m_old, warp_max(s));
          const float ps = warp_sum(valid ? expf(s - m_new) : 0.f);
          if (lane == 0) {
            l_s[r] = l_s[r] * expf(m_old - m_new) + ps;
            m_s[r] = m_new;
          }
        }
        continue;
      }
      // final weights of every head (l_s holds 1 / sum), then their mix over heads; no rescaling of the sums
      for (int idx = tid; idx < R * BK; idx += kThreads) {
        const int r = idx / BK, jj = idx - r * BK, i = r / H;
        Ss[idx] = (i < n && sees(p, pos0 + i, j0 + jj)) ? expf(Ss[idx] - m_s[r]) * l_s[r] : 0.f;
      }
      __syncthreads();
      for (int r = warp; r < R; r += kWarps) {
        const int i = r / H, h = r - i * H;
        if (lane < BK) {
          const float* tk = Tk + h * H;
          const float* sr = Ss + (i * H) * BK + lane;
          float w = 0.f;
          for (int g = 0; g < H; ++g) w = fmaf(tk[g], sr[g * BK], w);
          Ps[r * BK + lane] = w;
        }
        if (lane == 0) a_s[r] = 1.0f;
      }
    } else
    // head mixing + mask + online softmax: a warp per score row, a lane per key
    for (int r = warp; r < R; r += kWarps) {
      const int i = r / H, h = r - i * H;
      const bool valid = lane < BK && i < n && sees(p, pos0 + i, j0 + lane);
      float s = 0.f;
      if (lane < BK) {
        const float* tk = Tk + h * H;
        const float* sr = Ss + (i * H) * BK + lane;
        for (int g = 0; g < H; ++g) s = fmaf(tk[g], sr[g * BK], s);
      }
      if (valid && p.dist_bias) s += dist_bias(p, pos0 + i - (j0 + lane), h);
      s = valid ? s : kNegBig;
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float pj = valid ? expf(s - m_new) : 0.f;
      const float ps = warp_sum(pj);
      if (lane < BK) Ps[r * BK + lane] = pj;
      if (lane == 0) {
        const float alpha = expf(m_old - m_new);
        a_s[r] = alpha;
        l_s[r] = l_s[r] * alpha + ps;
        m_s[r] = m_new;
      }
    }
    __syncthreads();
    // weighted sum of the values
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int o = tid + a * kThreads;
      if (o < nout) {
        const int r = o / vq, c4 = o - r * vq, h = r % H;
        const float alpha = a_s[r];
        float4 v = acc[a];
        v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
        const float* pr = Ps + r * BK;
        const float* vr = Vs + (h / rep) * V4 + 4 * c4;
        for (int jj = 0; jj < BK; ++jj) {
          const float pj = pr[jj];
          const float4 c = *reinterpret_cast<const float4*>(vr + jj * G * V4);
          v.x = fmaf(pj, c.x, v.x); v.y = fmaf(pj, c.y, v.y); v.z = fmaf(pj, c.z, v.z); v.w = fmaf(pj, c.w, v.w);
        }
        acc[a] = v;
      }
    }
  }
  }
  __syncthreads();
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int o = tid + a * kThreads;
    if (o >= nout) continue;
    const int r = o / vq, c4 = o - r * vq, i = r / H, h = r - i * H;
    if (i >= n) continue;
    const float v[4] = {acc[a].x, acc[a].y, acc[a].z, acc[a].w};
    if (nsplit == 1) {
      const float inv = after ? out_gate(p, row0 + i, h) : out_gate(p, row0 + i, h) / l_s[r];
      const size_t ob = (static_cast<size_t>(row0 + i) * H + h) * V + 4 * c4;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (4 * c4 + e < V) st_any(p.out, p.out_dtype, ob + e, v[e] * inv);
    } else {
      float* part = p.partial + ((static_cast<size_t>(row0 + i) * nsplit + split) * H + h) * (V + 2);
      if (!(after && sh.phase == 0)) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (4 * c4 + e < V) part[4 * c4 + e] = v[e];
      }
      // with the weights mixed afterwards the (max, sum) slots belong to the first launch: the second one reads them
      if (c4 == 0 && !(after && sh.phase == 1)) { part[V] = m_s[r]; part[V + 1] = l_s[r]; }
    }
  }
}

// Prompt portions: BQ (a multiple of 4) rows x all heads per CTA, register-tiled.  Score rows are ordered
// head-major (r = h * BQ + i) so that 4 consecutive score rows are 4 query rows of ONE head: they share
// the key / value head, and a thread that owns such a block of 4 keeps
//   scores:        TR (4, or 2 with 512 threads) rows x 2 keys (jp and jp + BK / 2) per thread, q and k as float4
//                  pieces: 6 shared loads per 32 multiply-adds (4 per 16)
//   weighted sum:  4 rows x 4 value columns per accumulator, the 4 weights of a key as ONE float4
//                  (Ps is [row block][key][4]): 2 shared loads per 16 multiply-adds
// Shared memory (floats): Qs [R][D4] | Ks [BK][G][DS] | Vs [BK][G][V4] | Ss [R][BK] | Ps [R / 4][BK][4] |
//   m, l, alpha [R] | talk [H * H]
template <int NACC, int NT, int TR>
__global__ void __launch_bounds__(NT) paged_attn_tile4_kernel(const vila_paged_attn_params p, const AttnShape sh) {
  extern __shared__ __align__(16) float sm[];
  // H, G: the heads this CTA serves (all of them, or one K/V head with its query heads: global heads h0 + h, g0 + g)
  const int H = p.H / sh.hsplit, G = p.G / sh.hsplit, h0 = blockIdx.z * H, g0 = blockIdx.z * G;
  const int D = p.dim, V = p.vdim, BQ = sh.BQ, BK = sh.BK, HK = sh.BK >> 1;
  const int D4 = round4(D), DS = D4 + 4, V4 = round4(V), R = BQ * H, NB = R >> 2, rep = H / G, KS = key_stride(G, DS);
  float* Qs = sm;
  float* Ks = Qs + R * D4;
  float* Vs = Ks + BK * KS;
  float* Ss = Vs + BK * G * V4;
  float* Ps = Ss + R * BK;
  float* m_s = Ps + R * BK;
  float* l_s = m_s + R;
  float* a_s = l_s + R;
  float* Tk = a_s + R;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int i0 = blockIdx.y * BQ;
  const int n_tile = tile[1];
  if (i0 >= n_tile) return;
  const int row0 = tile[0] + i0, n = min(BQ, n_tile - i0), pos0 = tile[2] + i0;
  const int32_t* pt = p.page_tables + static_cast<size_t>(tile[3]) * p.pt_stride;

  for (int idx = tid; idx < R * D4; idx += NT) {
    const int r = idx / D4, k = idx - r * D4, h = r / BQ, i = r - h * BQ;
    Qs[idx] = (i < n && k < D) ? p.q[(static_cast<size_t>(row0 + i) * p.H + h0 + h) * D + k] * head_scale(p, h0 + h) : 0.f;
  }
  for (int idx = tid; idx < H * H; idx += NT) Tk[idx] = p.talk ? p.talk[idx] : ((idx / H) == (idx % H) ? 1.f : 0.f);
  const bool after = p.talk_after != 0 && p.talk != nullptr;
  for (int r = tid; r < R; r += NT) {
    const bool sink = p.sink != nullptr && !after;
    m_s[r] = sink ? p.sink[h0 + r / BQ] : kNegBig;
    l_s[r] = sink ? 1.0f : 0.0f;
  }
  float4 acc[NACC][4];
#pragma unroll
  for (int a = 0; a < NACC; ++a)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[a][k] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int vq = V4 >> 2;
  const int nout = NB * vq;               // accumulator items of the CTA: o -> (row block, float4 column)
  const int nkeys = pos0 + n;
  const int d4n = D4 >> 2;

  const BlockList bl = visible_blocks(p, pos0, nkeys, BK);
  for (int pass = after ? 0 : 1; pass < 2; ++pass) {
  const bool stats = pass == 0;   // scores only: every head's running max and sum over all visible keys
  if (after && !stats) {
    __syncthreads();
    for (int r = tid; r < R; r += NT) l_s[r] = l_s[r] > 0.f ? 1.0f / l_s[r] : 0.f;
  }
  for (int vb_ = 0; vb_ < bl.count; ++vb_) {
    const int j0 = bl.block(vb_) * BK;
    __syncthreads();
    load_kv_block(Ks, Vs, p, pt, j0, nkeys, BK, D4, DS, V4, NT / 32, g0, G, !stats);
    __syncthreads();
    for (int item = tid; item < (R / TR) * HK; item += NT) {
      const int rbs = item / HK, jp = item - rbs * HK, r0 = rbs * TR;     // TR score rows of one head x 2 keys
      const int g = (r0 / BQ) / rep;
      const float4* q0 = reinterpret_cast<const float4*>(Qs + r0 * D4);
      const float4* k0 = reinterpret_cast<const float4*>(Ks + jp * KS + g * DS);
      const float4* k1 = reinterpret_cast<const float4*>(Ks + (jp + HK) * KS + g * DS);
      float s[TR][2];
#pragma unroll
      for (int a = 0; a < TR; ++a) s[a][0] = s[a][1] = 0.f;
#pragma unroll 2
      for (int k = 0; k < d4n; ++k) {
        const float4 ka = k0[k], kb = k1[k];
#pragma unroll
        for (int a = 0; a < TR; ++a) {
          const float4 qv = q0[a * d4n + k];
          s[a][0] = fmaf(qv.x, ka.x, s[a][0]); s[a][0] = fmaf(qv.y, ka.y, s[a][0]);
          s[a][0] = fmaf(qv.z, ka.z, s[a][0]); s[a][0] = fmaf(qv.w, ka.w, s[a][0]);
          s[a][1] = fmaf(qv.x, kb.x, s[a][1]); s[a][1] = fmaf(qv.y, kb.y, s[a][1]);
          s[a][1] = fmaf(qv.z, kb.z, s[a][1]); s[a][1] = fmaf(qv.w, kb.w, s[a][1]);
        }
      }
#pragma unroll
      for (int a = 0; a < TR; ++a) {
        Ss[(r0 + a) * BK + jp] = s[a][0];
        Ss[(r0 + a) * BK + jp + HK] = s[a][1];
      }
    }
    __syncthreads();
    if (after) {
      if (stats) {
        for (int r = warp; r < R; r += NT / 32) {
          const int i = r % BQ;
          const bool valid = lane < BK && i < n && sees(p, pos0 + i, j0 + lane);
          const float s = valid ? Ss[r * BK + lane] : kNegBig;
          const float m_old = m_s[r];
          const float m_new = fmaxf(m_old, warp_max(s));
          const float ps = warp_sum(valid ? expf(s - m_new) : 0.f);
          if (lane == 0) {
            l_s[r] = l_s[r] * expf(m_old - m_new) + ps;
            m_s[r] = m_new;
          }
        }
        continue;
      }
      for (int idx = tid; idx < R * BK; idx += NT) {
        const int r = idx / BK, jj = idx - r * BK, i = r % BQ;
        Ss[idx] = (i < n && sees(p, pos0 + i, j0 + jj)) ? expf(Ss[idx] - m_s[r]) * l_s[r] : 0.f;
      }
      __syncthreads();
      for (int r = warp; r < R; r += NT / 32) {
        const int h = r / BQ, i = r - h * BQ;
        if (lane < BK) {
          const float* tk = Tk + h * H;
          const float* sr = Ss + i * BK + lane;
          float w = 0.f;
          for (int g = 0; g < H; ++g) w = fmaf(tk[g], sr[g * BQ * BK], w);
          Ps[(((r >> 2) * BK + lane) << 2) + (r & 3)] = w;
        }
        if (lane == 0) a_s[r] = 1.0f;
      }
    } else
    // head mixing + mask + online softmax: a warp takes 4 score rows at a time (rows warp, warp + 8, ...), a
    // lane per key; the 4 rows' reductions are interleaved so that their shuffles overlap
    for (int rbase = warp; rbase < R; rbase += 4 * (NT / 32)) {
      float sv[4], mo[4], mn[4], pj[4], ps[4];
      bool ok[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rbase + u * (NT / 32);
        sv[u] = kNegBig;
        ok[u] = false;
        mo[u] = kNegBig;
        if (r < R) {
          const int h = r / BQ, i = r - h * BQ;
          ok[u] = lane < BK && i < n && sees(p, pos0 + i, j0 + lane);
          if (lane < BK) {
            const float* tk = Tk + h * H;
            const float* sr = Ss + i * BK + lane;
            float s0 = 0.f, s1 = 0.f;
            int g = 0;
            for (; g + 1 < H; g += 2) {
              s0 = fmaf(tk[g], sr[g * BQ * BK], s0);
              s1 = fmaf(tk[g + 1], sr[(g + 1) * BQ * BK], s1);
            }
            if (g < H) s0 = fmaf(tk[g], sr[g * BQ * BK], s0);
            if (ok[u]) sv[u] = s0 + s1 + (p.dist_bias ? dist_bias(p, pos0 + i - (j0 + lane), h0 + h) : 0.f);
          }
          mo[u] = m_s[r];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) mn[u] = sv[u];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < 4; ++u) mn[u] = fmaxf(mn[u], __shfl_xor_sync(0xffffffffu, mn[u], o));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        mn[u] = fmaxf(mn[u], mo[u]);
        pj[u] = ok[u] ? expf(sv[u] - mn[u]) : 0.f;
        ps[u] = pj[u];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < 4; ++u) ps[u] += __shfl_xor_sync(0xffffffffu, ps[u], o);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rbase + u * (NT / 32);
        if (r < R) {
          if (lane < BK) Ps[(((r >> 2) * BK + lane) << 2) + (r & 3)] = pj[u];
          if (lane == 0) {
            const float alpha = expf(mo[u] - mn[u]);
            a_s[r] = alpha;
            l_s[r] = l_s[r] * alpha + ps[u];
            m_s[r] = mn[u];
          }
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int o = tid + a * NT;
      if (o < nout) {
        const int rb = o / vq, c4 = o - rb * vq;
        const int g = ((rb << 2) / BQ) / rep;
        const float4 al = *reinterpret_cast<const float4*>(a_s + (rb << 2));
        const float alv[4] = {al.x, al.y, al.z, al.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[a][k].x *= alv[k]; acc[a][k].y *= alv[k]; acc[a][k].z *= alv[k]; acc[a][k].w *= alv[k];
        }
        const float4* pr = reinterpret_cast<const float4*>(Ps + ((rb * BK) << 2));
        const float* vr = Vs + g * V4 + 4 * c4;
#pragma unroll 4
        for (int jj = 0; jj < BK; ++jj) {
          const float4 pw = pr[jj];
          const float4 c = *reinterpret_cast<const float4*>(vr + jj * G * V4);
          const float pv[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            acc[a][k].x = fmaf(pv[k], c.x, acc[a][k].x); acc[a][k].y = fmaf(pv[k], c.y, acc[a][k].y);
            acc[a][k].z = fmaf(pv[k], c.z, acc[a][k].z); acc[a][k].w = fmaf(pv[k], c.w, acc[a][k].w);
          }
        }
      }
    }
  }
  }
  __syncthreads();
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    const int o = tid + a * NT;
    if (o >= nout) continue;
    const int rb = o / vq, c4 = o - rb * vq;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int r = (rb << 2) + k, h = r / BQ, i = r - h * BQ;
      if (i >= n) continue;
      const float inv = after ? out_gate(p, row0 + i, h0 + h) : out_gate(p, row0 + i, h0 + h) / l_s[r];
      const float v[4] = {acc[a][k].x, acc[a][k].y, acc[a][k].z, acc[a][k].w};
      const size_t ob = (static_cast<size_t>(row0 + i) * p.H + h0 + h) * V + 4 * c4;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (4 * c4 + e < V) st_any(p.out, p.out_dtype, ob + e, v[e] * inv);
    }
  }
}

// one CTA per (decoded row, head): combine the nsplit partial triples in split order
__global__ void __launch_bounds__(128) paged_attn_merge_kernel(const vila_paged_attn_params p) {
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row = tile[0], h = blockIdx.y, V = p.vdim, ns = p.nsplit;
  const float* part = p.partial + (static_cast<size_t>(row) * ns * p.H + h) * (V + 2);
  const size_t stride = static_cast<size_t>(p.H) * (V + 2);
  if (p.talk_after != 0 && p.talk != nullptr) {   // the partial sums carry final weights: add them in split order
    const float gt = out_gate(p, row, h);
    for (int k = threadIdx.x; k < V; k += blockDim.x) {
      float a = 0.f;
      for (int s = 0; s < ns; ++s) a += part[s * stride + k];
      st_any(p.out, p.out_dtype, (static_cast<size_t>(row) * p.H + h) * V + k, a * gt);
    }
    return;
  }
  float mx = kNegBig;
  for (int s = 0; s < ns; ++s) mx = fmaxf(mx, part[s * stride + V]);
  float den = 0.f;
  for (int s = 0; s < ns; ++s) den += expf(part[s * stride + V] - mx) * part[s * stride + V + 1];
  const float inv = out_gate(p, row, h) / den;
  for (int k = threadIdx.x; k < V; k += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < ns; ++s) a += expf(part[s * stride + V] - mx) * part[s * stride + k];
    st_any(p.out, p.out_dtype, (static_cast<size_t>(row) * p.H + h) * V + k, a * inv);
  }
}

size_t attn_smem(const vila_paged_attn_params& p, int BQ, int BK, int H = 0, int G = 0) {
  if (H == 0) { H = p.H; G = p.G; }
  const int D4 = round4(p.dim), V4 = round4(p.vdim), R = BQ * H;
  return sizeof(float) * (static_cast<size_t>(R) * D4 + static_cast<size_t>(BK) * key_stride(G, D4 + 4) +
                          static_cast<size_t>(BK) * G * V4 + 2 * static_cast<size_t>(R) * BK + H * H + 3 * R);
}

}  // namespace

int rope_append(const vila_rope_append_params& p, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  VB_CHECK(p.H >= 1 && p.G >= 1 && p.dim >= 1 && p.vdim >= 1 && p.rot_dims >= 0 && p.rot_dims <= p.dim &&
               p.rot_dims % 2 == 0 && (p.rot_dims == 0 || p.inv_freq != nullptr) && (!p.v_from_k || p.vdim == p.dim) &&
               (p.rot_layout == 0 || p.rot_layout == 1),
           "rope_append: H=%d G=%d dim=%d vdim=%d rot_dims=%d v_from_k=%d", p.H, p.G, p.dim, p.vdim, p.rot_dims,
           p.v_from_k);
  VB_CUDA(launch_serial(rope_append_kernel, dim3(p.T), dim3(kThreads), sizeof(float) * (p.rot_dims + 2), stream, p));
  return 0;
}

int paged_attention(const vila_paged_attn_params& p, cudaStream_t stream) {
  if (p.ntiles <= 0) return 0;
  VB_CHECK(p.H >= 1 && p.G >= 1 && p.H % p.G == 0 && p.dim >= 1 && p.vdim >= 1 && p.page >= 1 && p.nsplit >= 1 &&
               p.nsplit <= 64 && (p.nsplit == 1 || p.partial != nullptr),
           "paged_attention: H=%d G=%d dim=%d vdim=%d page=%d nsplit=%d", p.H, p.G, p.dim, p.vdim, p.page, p.nsplit);
  constexpr size_t kSmemMax = 224 * 1024;
  VB_CHECK(p.chunk >= 0 && (p.dist_bias == nullptr || p.dist_rows >= 1), "paged_attention: chunk=%d dist_rows=%d",
           p.chunk, p.dist_rows);
  VB_CHECK(p.window >= 0 && p.keep_first >= 0 && (p.talk_after == 0 || (p.talk != nullptr && p.sink == nullptr)),
           "paged_attention: window=%d keep_first=%d; talk_after needs talk and no sink", p.window, p.keep_first);
  VB_CHECK(p.max_rows >= 1 && p.max_rows <= 16 && (p.nsplit == 1 || p.max_rows == 1),
           "paged_attention: max_rows=%d nsplit=%d (key splitting serves one-row tiles)", p.max_rows, p.nsplit);
  AttnShape sh;
  sh.phase = -1;
  // Without head mixing the K/V-head groups are independent: a CTA then serves ONE K/V head and its query heads, holds
  // a quarter .. an eighth of the K | V block, and takes more rows of the sequence instead.
  sh.hsplit = (p.talk == nullptr && p.max_rows > 1) ? p.G : 1;
  const int Hl = p.H / sh.hsplit, Gl = p.G / sh.hsplit;
  if (p.max_rows > 1 && Hl <= 32) {
    // prompt portions: the register-tiled kernel, 4 .. 16 rows per CTA (about 64 score rows, 128 at most)
    sh.BQ = 16;
    while (sh.BQ > 4 && sh.BQ * Hl > 64) sh.BQ >>= 1;
    sh.BK = 32;
    while (attn_smem(p, sh.BQ, sh.BK, Hl, Gl) > kSmemMax && sh.BK > 8) sh.BK >>= 1;
    const size_t smem4 = attn_smem(p, sh.BQ, sh.BK, Hl, Gl);
    const int items = (sh.BQ * Hl / 4) * (round4(p.vdim) >> 2);      // accumulator items (4 rows x 4 columns)
    // 512 threads (16 warps on the SM, 2-row score tiles) when there is accumulator work for them
    const int nt = items >= 512 ? 512 : 256;
    const int nacc4 = (items + nt - 1) / nt;
    if (smem4 <= kSmemMax && nacc4 <= (nt == 512 ? 2 : 4)) {
      sh.sub = (p.max_rows + sh.BQ - 1) / sh.BQ;
      const dim3 grid4(p.ntiles, sh.sub, sh.hsplit);
#define VB_PAGED4(N, NT, TR)                                                                                     \
  do {                                                                                                           \
    if (smem4 > 48 * 1024)                                                                                       \
      VB_CUDA(cudaFuncSetAttribute(paged_attn_tile4_kernel<N, NT, TR>,                                           \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem4)));       \
    VB_CUDA(launch_serial(paged_attn_tile4_kernel<N, NT, TR>, grid4, dim3(NT), smem4, stream, p, sh));           \
  } while (0)
      if (nt == 512) {
        if (nacc4 <= 1) VB_PAGED4(1, 512, 2);
        else VB_PAGED4(2, 512, 2);
      } else if (nacc4 <= 1) VB_PAGED4(1, 256, 4);
      else if (nacc4 <= 2) VB_PAGED4(2, 256, 4);
      else VB_PAGED4(4, 256, 4);
#undef VB_PAGED4
      return 0;
    }
  }
  // decoded tokens (one-row tiles, keys optionally split over CTAs) and shapes the tiled kernel does not take
  sh.hsplit = 1;
  sh.BQ = 1;
  while (sh.BQ < p.max_rows) sh.BQ <<= 1;
  while (sh.BQ > 1 && sh.BQ * p.H > 64) sh.BQ >>= 1;
  sh.BK = 32;
  while (attn_smem(p, sh.BQ, sh.BK) > kSmemMax && sh.BK > 4) sh.BK >>= 1;
  while (attn_smem(p, sh.BQ, sh.BK) > kSmemMax && sh.BQ > 1) sh.BQ >>= 1;
  const size_t smem = attn_smem(p, sh.BQ, sh.BK);
  VB_CHECK(smem <= kSmemMax, "paged_attention: H=%d G=%d dim=%d vdim=%d need %zu bytes of shared memory", p.H, p.G,
           p.dim, p.vdim, smem);
  sh.sub = (p.max_rows + sh.BQ - 1) / sh.BQ;
  const int nacc = (sh.BQ * p.H * (round4(p.vdim) >> 2) + kThreads - 1) / kThreads;
  VB_CHECK(nacc <= 16, "paged_attention: H=%d vdim=%d: %d accumulators per thread", p.H, p.vdim, nacc);
  const dim3 grid(p.ntiles, sh.sub, p.nsplit);
#define VB_PAGED(N)                                                                                              \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      VB_CUDA(cudaFuncSetAttribute(paged_attn_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                   static_cast<int>(smem)));                                                     \
    VB_CUDA(launch_serial(paged_attn_kernel<N>, grid, dim3(kThreads), smem, stream, p, sh));                     \
  } while (0)
  // weights mixed after the softmax + split keys: the (max, sum) launch, then the launch that adds the values
  const int launches = (p.talk_after != 0 && p.nsplit > 1) ? 2 : 1;
  for (int l = 0; l < launches; ++l) {
    sh.phase = launches == 2 ? l : -1;
    if (nacc <= 1) VB_PAGED(1);
    else if (nacc <= 2) VB_PAGED(2);
    else if (nacc <= 4) VB_PAGED(4);
    else if (nacc <= 8) VB_PAGED(8);
    else VB_PAGED(16);
  }
#undef VB_PAGED
  if (p.nsplit > 1)
    VB_CUDA(launch_serial(paged_attn_merge_kernel, dim3(p.ntiles, p.H), dim3(128), 0, stream, p));
  return 0;
}

}  // namespace vb
