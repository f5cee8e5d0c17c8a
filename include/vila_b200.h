/*
 * vila_b200 — C-ABI of the B200-native (sm_100a) VILA multimodal forward hot path.
 *
 * The reference (NVlabs/VILA) has no FFI on this path: every GPU op is a library call made from
 * Python (flash_attn, cuBLAS through nn.Linear, cuDNN through nn.Conv2d, ATen elementwise).  This
 * header is the boundary a maintainer would bind instead of those calls; each entry point names the
 * reference call site (paths relative to the VILA repo root) it replaces.  The only native-extension
 * precedent in the tree (llava/model/coat/optimizer/kernels/bindings.cpp:6-10) takes tensors,
 * mutates in place, returns void and runs on the current stream; we keep "caller owns all memory,
 * in-place/out-param, stream-ordered", but with plain pointers so any host language can bind it.
 *
 * Conventions
 *   - all tensor pointers are DEVICE pointers to bf16 (uint16 storage) unless stated otherwise,
 *     row-major, 16-byte aligned; leading dimensions are in ELEMENTS;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - every function returns 0 on success; non-zero on error, message via vila_last_error()
 *     (thread-local). Nothing falls back to the CPU: without an sm_100a device calls fail.
 *   - no hidden state beyond (a) the per-device stream-K scratch registered with vila_set_workspace and
 *     (b) per-device "function attributes set" flags: KV pool, page tables, workspaces and counters
 *     are caller-allocated.
 */
#ifndef VILA_B200_H_
#define VILA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VILA_ACT_NONE 0
#define VILA_ACT_GELU_TANH 1 /* SigLIP "gelu_pytorch_tanh"  (modeling_siglip.py:707-715) */
#define VILA_ACT_GELU_ERF 2  /* nn.GELU() in mm_projector   (base_projector.py:145-162)  */
#define VILA_ACT_SILU 3

/* `flags` of vila_linear / vila_gemv:
 *   VILA_FLAG_SWIGLU    weight rows are interleaved (gate_0, up_0, gate_1, ...); out is [M, N/2] =
 *                       silu(gate) * up
 *   VILA_FLAG_STATIC_W  the weight matrix is a parameter that no earlier kernel in this stream is
 *                       still writing: the kernel may fetch it BEFORE the programmatic-dependent-launch
 *                       wait (all vila_* kernels are launched with PDL so that prologues and weight
 *                       prefetch overlap the predecessor's tail). Leave it clear for weights produced
 *                       on the fly. */
#define VILA_FLAG_SWIGLU 1
#define VILA_FLAG_STATIC_W 2

const char* vila_last_error(void);
int vila_abi_version(void); /* 3 */
/* Register caller-owned, ZERO-INITIALISED device scratch (256-byte aligned) used by vila_linear's
 * stream-K schedule for fp32 partial sums (64 KiB of counters + M*N*4 bytes per call that uses it;
 * calls that do not fit simply use the data-parallel schedule).  The kernels leave it zeroed again.
 * The registration is per DEVICE (the current device at the time of the call); one workspace serves
 * one stream at a time.  ptr == NULL unregisters. */
int vila_set_workspace(void* ptr, uint64_t bytes);
/* fills SM count and compute capability of the current device */
int vila_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* ---------------------------------------------------------------------------------------------
 * vila_linear — out[M,N] = epilogue(x[M,K] · w[N,K]^T)        (tcgen05 / TMEM / TMA GEMM)
 *   epilogue: (+bias[N]) -> act -> (+residual[row % res_row_mod or row, :])   or SwiGLU:
 *   flags & VILA_FLAG_SWIGLU: w rows are interleaved (gate_0, up_0, gate_1, up_1, ...) and out is
 *   [M, N/2] = silu(gate) * up.
 * Replaces nn.Linear (+ the ATen GELU / SiLU*mul / residual add that follows it):
 *   SigLIP q/k/v/out_proj, fc1/fc2 : llava/model/multimodal_encoder/siglip/modeling_siglip.py:384-387,707-715,752,757
 *   patch-embed Conv2d (as im2col GEMM, residual = position embedding with res_row_mod = #patches): :269-275,322-328
 *   mm_projector Linear layers     : llava/model/multimodal_projector/base_projector.py:145-162
 *   Qwen2 q/k/v/o, gate/up/down, lm_head: transformers Qwen2 (in-tree copy
 *     llava/eval/vision_niah_vila/zigzag_ring_attn/modeling_qwen2.py:164-176,223-226,633-706)
 * ------------------------------------------------------------------------------------------- */
int vila_linear(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias,
                const void* residual, int64_t ld_res, int res_row_mod, void* out, int64_t ldo,
                int M, int N, int K, int act, int flags, void* stream);
/* vila_linear with the coefficients of a two-parameter activation (VILA_ACT_XIELU: act_pos, act_neg); no residual. */
int vila_linear_act(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias, void* out, int64_t ldo,
                    int M, int N, int K, int act, float act_pos, float act_neg, int flags, void* stream);
/* test hook: same, forcing the kernel configuration instead of the size heuristic:
 *   64 / 128 / 256   single-CTA tiles 128 x block_n (+1000: deterministic stream-K, +2000: stream-K off)
 *   4128 / 4256      CTA-pair tiles 256 x {128,256} (tcgen05 cta_group::2)
 *   5128             split-K CTA pairs on 128 x 128 tiles (needs <= #SM/2 tiles, K > 64)
 *   3000 / 3001      swap-AB skinny kernel (M <= 512), one CTA / CTA pair per weight block */
int vila_linear_cfg(int block_n, const void* x, int64_t ldx, const void* w, int64_t ldw,
                    const void* bias, const void* residual, int64_t ld_res, int res_row_mod,
                    void* out, int64_t ldo, int M, int N, int K, int act, int flags, void* stream);

/* nn.LayerNorm over the last dim (modeling_siglip.py:723,725,746,755; base_projector.py:147) */
int vila_layernorm(const void* x, const void* weight, const void* bias, void* out, int rows,
                   int cols, float eps, void* stream);
/* Qwen2RMSNorm (modeling_qwen2.py:81-95). If residual_add != NULL: x += residual_add first (in place). */
int vila_rmsnorm(void* x_inout, const void* residual_add, const void* weight, void* out, int rows,
                 int cols, float eps, void* stream);

/* ---------------------------------------------------------------------------------------------
 * vila_fmha — flash attention forward, tcgen05 QK^T / PV with TMEM accumulators.
 *   q/o element (token t, head h, dim d) at  base + t*tok_stride + h*head_stride + d
 *   k/v: if kv_page_stride != 0 the KV cache is paged (128 tokens per page):
 *          element (page p, row r, head h, d) at base + p*kv_page_stride + r*kv_tok_stride + h*kv_head_stride + d
 *          and page_table[b*page_table_stride + j] gives the page of block j (NULL: identity);
 *        else k/v are [B*Sk, Hkv, D] views like q.
 * Replaces flash_attn_func(q,k,v,causal=False) in SiglipFlashAttention2 (modeling_siglip.py:583-585)
 * and HF _flash_attention_forward for Qwen2/Llama (patched at llava/train/sequence_parallel/
 * monkey_patch.py:133-239, llava/model/utils/packing.py:36), causal GQA.
 * ------------------------------------------------------------------------------------------- */
typedef struct vila_fmha_params {
  const void* q;
  int64_t q_tok_stride, q_head_stride;
  const void* k;
  const void* v;
  int64_t kv_page_stride, kv_tok_stride, kv_head_stride, kv_num_pages;
  const int32_t* page_table;
  int32_t page_table_stride;
  void* o;
  int64_t o_tok_stride, o_head_stride;
  int32_t B, Sq, Sk, Hq, Hkv, D, causal;
  float scale;
} vila_fmha_params;
int vila_fmha(const vila_fmha_params* p, void* stream);
/* test hook (like vila_linear_cfg): same, forcing the kernel flavour instead of the size heuristic:
 *   0 heuristic; 1 one query tile per CTA (fmha_fwd_kernel); 2 two query tiles per CTA with ping-pong
 *   softmax warpgroups and the O accumulator in TMEM (fmha2_fwd_kernel; needs Sq > 128, D in 72..96 or 128);
 *   3 / 4: as 2 with every 4th / every 2nd exponential as an FMA-pipe polynomial (measured slower) */
int vila_fmha_cfg(int variant, const vila_fmha_params* p, void* stream);

/* im2col for Conv2d(3,1152,k=14,s=14) (modeling_siglip.py:269-275): pixels [B,C,H,W] ->
 * out [B*(H/P)*(W/P), k_pad], column = (c, ky, kx); columns >= C*P*P are zero. */
int vila_patch_im2col(const void* pixels, void* out, int B, int C, int H, int W, int patch,
                      int k_pad, void* stream);
/* Image preprocessing on the device.  Replaces, per resize grid of
 * mm_utils.process_image (llava/mm_utils.py:442-522; dynamic_preprocess :299-338, dynamic_s2_preprocess
 * :341-405), PIL `image.resize((out_w, out_h))` (bicubic; Pillow Resample.c 8bpc fixed point) + the crop
 * into tile x tile blocks + SiglipImageProcessor.preprocess (rescale 1/255, normalise (x-mean)/std):
 *   src      uint8 [H, W, 3] (device)      tmp  uint8 scratch [H, out_w, 3]
 *   coef_*   int32 [out, ksize] 22-bit filter taps, bounds_* int32 [out, 2] = (first input index, count)
 *            (host: vila_b200.model.media.bicubic_coeffs == Pillow precompute_coeffs/normalize_coeffs_8bpc)
 *   out      bf16 [n_tiles, 3, tile, tile]; pixel (Y, X) of the resized image lands in tile
 *            tile_index0 + (Y / tile) * (out_w / tile) + X / tile.  Bit-identical to the PIL path. */
int vila_resize_bicubic_tiles(const uint8_t* src, int H, int W, int out_w, int out_h,
                              const int32_t* coef_x, const int32_t* bounds_x, int ksize_x,
                              const int32_t* coef_y, const int32_t* bounds_y, int ksize_y, uint8_t* tmp,
                              void* out_tiles, int tile, int tile_index0, float mean, float stdv,
                              void* stream);
/* DownSampleBlock.flat_square / flat_square_2x2 / flat_square_3x3 (base_projector.py:58-123):
 * x [B, h*w, C] -> out [B, ceil(h/r)*ceil(w/r), r*r*C], zero padded. */
int vila_space_to_depth(const void* x, void* out, int B, int h, int w, int C, int r, void* stream);
/* merge_features_for_dynamic_s2 + split_chessboard for one image (llava_arch.py:282-364). */
int vila_s2_merge(const void* tiles, void* out, int side, int C, int n_scales,
                  const int* splits_h, const int* splits_w, int out_bh, int out_bw, int share_tile,
                  void* stream);
/* merge_chessboard + "(h w) c" flatten of projected tiles (llava_arch.py:255-280,384-390). */
int vila_chessboard_merge(const void* tiles, void* out, int bh, int bw, int s, int C, void* stream);
/* TSPVideoEncoder pooling (llava/model/encoders/video/tsp.py:11-12,28-51). */
int vila_tsp_pool(const void* x, void* out, int T, int h, int w, int C, int pt, int ph, int pw,
                  void* stream);
/* text/media embedding splice of LlavaMetaForCausalLM._embed (llava_arch.py:429,457-479):
 * out[i] = src[i] >= 0 ? table[src[i]] : media[-(src[i]+1)].  src is int32 on the device. */
int vila_embed_splice(const void* table, const void* media, const int32_t* src, void* out, int rows,
                      int cols, void* stream);
/* HF apply_rotary_pos_emb (modeling_qwen2.py:99-160) in place on q,k of qkv [S,(Hq+2Hkv)*D] and
 * DynamicCache.update as a scatter into the paged pool (k_pool may be NULL: RoPE only).
 * inv_freq: fp32 [D/2] on the device. positions: int32 [S] on the device. */
int vila_rope_kv_append(void* qkv, const int32_t* positions, int S, int Hq, int Hkv, int D,
                        const float* inv_freq, void* k_pool, void* v_pool,
                        const int32_t* page_table, int cache_pos0, void* stream);
/* (cache_pos0 < 0: the cache slot of row s is positions[s] itself — decode, position on the device) */
/* vila_rope_kv_append with cos / sin taken from vila_rope_table(positions) (computed once per request
 * and shared by all layers and heads; 16-byte accesses): the long-prefill form, bit-identical. */
int vila_rope_kv_append_table(void* qkv, const void* rope_table, int S, int Hq, int Hkv, int D,
                              void* k_pool, void* v_pool, const int32_t* page_table, int cache_pos0,
                              void* stream);
/* Fused q/k/v projection for a short prefill chunk (M <= 384 tokens, head_dim 128):
 * qkv = x @ w^T + bias; RoPE on the q and k heads; q heads -> qkv_out[:, :Hq*128]; k / v heads ->
 * the paged pools (k_pool NULL: they stay in qkv_out) — vila_linear followed by vila_rope_kv_append
 * in ONE kernel, bit-identical to the two calls (rope_table: vila_rope_table of the chunk's positions).  Replaces Qwen2Attention's q_proj/k_proj/v_proj +
 * apply_rotary_pos_emb + past_key_value.update (modeling_qwen2.py:223-226,99-160,262-266 of the
 * in-tree copy).  Returns 3 (and sets vila_last_error) when the shape is not covered: the caller
 * then issues the two separate calls. */
int vila_linear_qkv_rope(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias,
                         void* qkv_out, int64_t ldo, int M, int K, int Hq, int Hkv, int D,
                         const void* rope_table, void* k_pool, void* v_pool,
                         const int32_t* page_table, int cache_pos0, int flags, void* stream);
/* cos / sin table of Qwen2RotaryEmbedding.forward (modeling_qwen2.py:99-143) for one request,
 * computed once and shared by all layers: table [S, D] bf16 = cos(pos*inv_freq[0..D/2)) | sin(...). */
int vila_rope_table(const int32_t* positions, int S, int D, const float* inv_freq, void* table,
                    void* stream);

/* ---------------------------------------------------------------------------------------------
 * decode (one token): weight-streaming GEMV with fused RMSNorm prologue and bias / residual /
 * SwiGLU / greedy-argmax epilogues; split-KV paged GQA attention with fused RoPE + KV append.
 * ------------------------------------------------------------------------------------------- */
typedef struct vila_gemv_params {
  const void* x;
  const void* w;
  const void* bias;
  const void* norm_w;
  float norm_eps;
  const void* residual;
  void* y;
  int32_t N, K;
  int32_t flags; /* VILA_FLAG_SWIGLU: rows interleaved (gate, up), y is [N/2];
                    VILA_FLAG_STATIC_W: see below */
  unsigned long long* argmax_key; /* device u64, zero before the first launch */
} vila_gemv_params;
int vila_gemv(const vila_gemv_params* p, void* stream);

int vila_argmax_finalize(unsigned long long* key, int32_t* token_out, int32_t* token_hist,
                         int32_t* step_counter, int32_t* position, const void* embed_table,
                         void* x_next, int hidden, void* stream);

typedef struct vila_decode_attn_params {
  void* qkv;
  const int32_t* position;
  void* k_pool;
  void* v_pool;
  const int32_t* page_table;
  void* out;
  float* ws;         /* >= Hkv*num_splits*G*(D+2) floats */
  int32_t* counters; /* Hkv ints, zero-initialised once */
  const float* inv_freq;
  int32_t Hq, Hkv, D, num_splits; /* num_splits 0: one CTA per query head, no split: the cache holds at
                                     most 1024 tokens (page_table has >= 8 entries); 1..8: KV splits as a
                                     thread-block cluster; 9..64: splits combined through ws/counters */
  float scale;
} vila_decode_attn_params;
int vila_decode_attention(const vila_decode_attn_params* p, void* stream);

/* Batched decode attention for continuous batching over ONE shared paged pool: `batch` sequences, sequence
 * b uses qkv + b*qkv_stride, out + b*out_stride, position[b] (< 0: idle slot, skipped) and the page-table
 * row page_table + b*pt_stride (max_pages <= 32 valid entries: contexts up to 4096 tokens).  ws / counters /
 * num_splits of the struct are ignored.  One CTA per (query head, sequence); RoPE + KV append fused. */
int vila_decode_attention_batch(const vila_decode_attn_params* p, int batch, int qkv_stride,
                                int out_stride, int pt_stride, int max_pages, void* stream);

/* Long-context decode attention (video: 16K-66K cached tokens = 34-135 MB of K/V per layer): RoPE +
 * KV append for the new token, then the tcgen05 FMHA kernel in split-KV mode (the G query heads of a
 * KV group are the query rows of its 128-row tile; K/V pages stream through TMA on
 * Hkv * num_splits CTAs), then a deterministic combine.  split j covers tokens
 * [j*split_tokens, (j+1)*split_tokens) (multiple of 128; num_splits*split_tokens >= max context).
 * Replaces the same HF calls as vila_decode_attention (apply_rotary_pos_emb + DynamicCache.update +
 * flash-attn decode, modeling_qwen2.py:99-160,262-310). */
typedef struct vila_decode_attn_split_params {
  void* qkv;
  const int32_t* position;
  void* k_pool;
  void* v_pool;
  const int32_t* page_table;
  int64_t kv_num_pages;
  void* out;
  float* o_partial; /* >= num_splits*Hq*D floats */
  float* lse;       /* >= num_splits*Hq floats */
  int32_t* counters; /* Hkv ints, zero before the first launch (self-cleaning): the last split CTA of a KV head
                        merges the partials itself; NULL: a separate combine kernel is launched */
  const float* inv_freq;
  int32_t Hq, Hkv, D, num_splits, split_tokens;
  float scale;
} vila_decode_attn_split_params;
int vila_decode_attention_split(const vila_decode_attn_split_params* p, void* stream);

/* ---------------------------------------------------------------------------------------------
 * vila_decode_mega — n_tokens greedy decode steps of the whole LLM in ONE persistent launch
 * (one CTA per SM, weights streamed through per-warp TMA rings that run ahead across layer and token
 * boundaries, grid barriers between phases).  Replaces the per-token HF generate loop
 * (llava_arch.py:833 -> GenerationMixin: ~400 launches and one D2H sync per token).
 * `layers` is a DEVICE array of num_layers entries.  `barrier` and `epoch` are device u32 words that
 * must both be zero before the first launch (the kernel keeps them consistent afterwards).
 * Head dim is 128.  The new tokens are appended to hist[*step ...], *position and *step advance.
 * ------------------------------------------------------------------------------------------- */
typedef struct vila_mega_layer {
  const void* qkv_w;
  const void* qkv_b;
  const void* o_w;
  const void* gu_w;
  const void* down_w;
  const void* ln1_w;
  const void* ln2_w;
  void* k_pool;
  void* v_pool;
} vila_mega_layer;
typedef struct vila_mega_params {
  const vila_mega_layer* layers;
  int32_t num_layers;
  const void* final_norm_w;
  const void* lm_head_w;
  const void* embed;
  int32_t hidden, inter, Hq, Hkv, vocab;
  float eps, scale;
  const float* inv_freq;
  const int32_t* page_table;
  void* x;
  void* qkv;
  void* act;
  float* attn_ws;
  int32_t* attn_counters; /* Hkv ints, zero before the first launch */
  unsigned long long* key;
  int32_t* token;
  int32_t* hist;
  int32_t* step;
  int32_t* position;
  uint32_t* barrier;
  uint32_t* epoch;
  int32_t n_tokens, splits;
} vila_mega_params;
int vila_decode_mega(const vila_mega_params* p, void* stream);

/* =============================================================================================
 * Ragged-batch building blocks of decoder-only language models that keep the residual stream in
 * fp32 (latent attention, gated linear recurrences, routed experts).  One step runs T token rows
 * taken from several sequences: a portion of one prompt next to single decoded tokens of others.
 * Every tensor argument carries a dtype code so the same kernels serve the bf16 serving path and
 * a true fp32 path:  VILA_DT_BF16 / VILA_DT_F32.  Sums, norms, softmax, gates and recurrent
 * state are always fp32.
 * ============================================================================================= */
#define VILA_DT_BF16 0
#define VILA_DT_F32 1
#define VILA_ACT_RELU2 4 /* max(z, 0)^2 */

/* out[t, :] = table[ids[t], :] as fp32 (the start of the fp32 residual stream) */
int vila_embed_rows(const void* table, int table_dtype, const int32_t* ids, float* out, int rows,
                    int cols, void* stream);

/* out[dst(r), :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * (w + w_offset)
 *   w_offset 1: weights stored around zero; 0: plain weights.  dst(r) = out_rows ? out_rows[r] : r
 *   (out_rows scatters the rows into a paged pool, e.g. a latent KV cache).  w may be NULL. */
int vila_rmsnorm_rows(const void* x, int x_dtype, int64_t ldx, const void* w, int w_dtype,
                      float w_offset, float eps, void* out, int out_dtype, int64_t ldo,
                      const int32_t* out_rows, int rows, int cols, void* stream);

/* Gated, normed residual update of the fp32 stream x [rows, cols]:
 *   y = sum_{j < n_partials} part[r * n_partials + j, :]          (fixed order)
 *   y = y * sigmoid(gate[r, :] + gate_bias)                        (gate == NULL: no gate)
 *   x[r, :] += y / sqrt(mean(y^2) + eps) * (w + w_offset)          (w == NULL: no norm weight) */
int vila_gated_norm_residual(float* x, const void* part, int part_dtype, int64_t ldp, int n_partials,
                             const void* gate, int gate_dtype, int64_t ldg, const void* gate_bias,
                             int bias_dtype, const void* w, int w_dtype, float w_offset, float eps,
                             int rows, int cols, void* stream);

/* vila_glinear — any-shape (grouped) linear layer on the CUDA cores with fp32 accumulation:
 *   out = act(a · w[g]^T + bias[g]) (* row_scale)
 * mode 0 (batched): every group g sees all M rows; its A columns start at g * a_group_off and its
 *   output columns at g * o_group_off (per-head projections); groups == 1 is a plain linear layer.
 * mode 1 (segmented): the rows of group g are the sorted positions [seg[g], seg[g+1]) (routed experts);
 *   position i reads A row a_rows[i] / a_row_div (a_rows NULL: i) and writes output row o_rows[i]
 *   (NULL: i), scaled by row_scale[o_rows[i]] when row_scale is given.  M bounds seg[groups].
 * flags: VILA_FLAG_SWIGLU as in vila_linear (out has N / 2 columns). */
typedef struct vila_glinear_params {
  const void* a;
  int64_t lda;
  const void* w;
  int64_t ldw, w_group_stride;
  const void* bias;
  int64_t bias_group_stride;
  void* out;
  int64_t ldo;
  int64_t a_group_off, o_group_off;
  const int32_t* seg;
  const int32_t* a_rows;
  const int32_t* o_rows;
  const float* row_scale;
  int32_t a_dtype, w_dtype, out_dtype;
  int32_t M, N, K, groups, mode, a_row_div, act, flags;
} vila_glinear_params;
int vila_glinear(const vila_glinear_params* p, void* stream);

/* vila_latent_attention — causal attention of H query heads over ONE shared latent per token
 * (keys and values are both the cached latent c_j of width R; the per-head key/value expansions
 * are folded into the queries before and into the output after this call):
 *   s_ij = scale * <q_i, c_j>,  j <= pos(i);   p_ij = exp(s_ij) / (sum_j exp(s_ij) + exp(sink_h))
 *   out_i = sigmoid(gate[i, h]) * sum_j p_ij c_j
 * sink == NULL: ordinary softmax; gate == NULL: no output gate.  The latent lives in pages of
 * `page` tokens: token j of a sequence is row page_tables[slot * pt_stride + j / page] * page + j % page.
 * tiles [ntiles, 4] = (first batch row, rows (<= 16), position of the first row, slot): consecutive
 * rows of one sequence.  decode != 0 selects the one-row-per-tile kernel (all rows must be 1); with
 * nsplit > 1 the 32-key blocks of a row are dealt round-robin to nsplit CTAs whose partial results
 * (partial: fp32 [T, H, nsplit, R + 2], caller-owned) are merged by a second kernel. */
typedef struct vila_latent_attn_params {
  const float* q; /* [T, H, R] */
  const void* cache;
  const int32_t* page_tables;
  const int32_t* tiles;
  const float* sink;
  const void* gate;
  void* out; /* [T, H, R] */
  float* partial;
  int64_t ldg;
  int32_t cache_dtype, gate_dtype, out_dtype;
  int32_t ntiles, pt_stride, H, R, page, decode, nsplit;
  float scale;
  int32_t window; /* > 0: row i sees the keys pos(i) - window < j <= pos(i) only; 0: all keys up to pos(i) */
} vila_latent_attn_params;
int vila_latent_attention(const vila_latent_attn_params* p, void* stream);

/* vila_latent_rope_append — what a latent-attention layer with a decoupled rotary part does between its
 * projections and vila_latent_attention (all fp32 arithmetic, angles in double):
 *   kv != NULL: pool row cache_rows[t] = rmsnorm(kv[t, :R]) * norm_w | rotate(kv[t, R : R + rot])
 *               (the normed latent and ONE rotated key part shared by all heads)
 *   q  != NULL: qa[t, h, R : R + rot] = rotate(q[t, h, q_off : q_off + rot])  for every head h, where
 *               head h of q starts at column h * q_head; qa rows are H * (R + rot) wide and their
 *               first R columns per head (the query with the key expansion folded in) are left alone.
 * rotate turns the pairs (2i, 2i+1) (layout 0) or (i, i + rot / 2) (layout 1) by positions[t] *
 * inv_freq[i] (fp64 [rot / 2]) and multiplies cos and sin by mscale. */
typedef struct vila_latent_rope_params {
  const void* kv; /* [T, ld_kv] or NULL */
  int64_t ld_kv;
  const float* norm_w; /* [R] or NULL */
  void* pool;          /* [pool rows, R + rot] */
  const int32_t* cache_rows;
  const void* q; /* [T, ld_q] or NULL */
  int64_t ld_q;
  float* qa; /* [T, H * (R + rot)] */
  const int32_t* positions;
  const double* inv_freq;
  int32_t kv_dtype, pool_dtype, q_dtype, T, H, R, rot, q_head, q_off, layout;
  float eps, mscale;
} vila_latent_rope_params;
int vila_latent_rope_append(const vila_latent_rope_params* p, void* stream);

/* vila_hgrn2_scan — gated linear recurrence with the forget gate tied to the input gate, per head:
 *   q_t = silu(zq_t),  f_t = lower + (1 - lower) * sigmoid(zf_t + f_bias)
 *   S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T   (S: [dim, vdim] fp32),   o_t = S_t^T q_t
 * proj holds zq | zf | v at column offsets q_off / f_off / v_off.  seqs [nseq, 4] = (first batch row,
 * rows, position of the first row, state slot); a sequence at position 0 starts from S = 0, otherwise
 * from state[slot]; the state after its last row is written back.  out [T, H * vdim] fp32. */
typedef struct vila_hgrn2_params {
  const void* proj;
  int64_t ldp;
  const float* f_bias;
  const float* lower;
  float* state; /* [slots, H, dim, vdim] */
  const int32_t* seqs;
  float* out;
  int32_t proj_dtype, q_off, f_off, v_off, nseq, H, dim, vdim;
} vila_hgrn2_params;
int vila_hgrn2_scan(const vila_hgrn2_params* p, void* stream);

/* Router of a mixture of experts: z = w_router x + bias in fp32, the `top` largest logits (ties: the
 * lower index), weights = softmax over the chosen logits.  idx / weight are [rows, top]. */
int vila_moe_route(const void* x, int x_dtype, int64_t ldx, const float* w_router, const float* bias,
                   int32_t* idx, float* weight, int rows, int cols, int experts, int top, void* stream);
/* Stable counting sort of the rows * top (token, choice) pairs by expert: seg [experts + 1] and
 * sorted [rows * top] (pair ids = row * top + choice), for vila_glinear mode 1. */
int vila_moe_group(const int32_t* idx, int32_t* seg, int32_t* sorted, int pairs, int experts,
                   void* stream);

/* dst[i, :] = src[rows[i], :] for rows of row_bytes bytes (any dtype; 16-byte copies when row_bytes and
 * both bases allow).  Used to lay the cached latents of a sequence out contiguously. */
int vila_gather_rows(const void* src, const int32_t* rows, void* dst, int n_rows, int row_bytes,
                     void* stream);

/* vila_sink_attention — causal multi-head attention with separate keys and values, fp32 scores /
 * softmax / weighted sum, optional per-head sink in the denominator and sigmoid output gate (as
 * vila_latent_attention).  k / v hold, for every sequence of the launch, the rows of ALL its positions
 * 0 .. pos0 + rows - 1, contiguously from row kv_row0: head h of position j at
 * k[(kv_row0 + j) * ldk + h * dim], v[(kv_row0 + j) * ldv + h * vdim].
 * tiles [ntiles, 4] = (first batch row, rows (<= 16), position of the first row, kv_row0). */
typedef struct vila_sink_attn_params {
  const void* q; /* [T, H * dim] */
  const void* k;
  const void* v;
  const int32_t* tiles;
  const float* sink;
  const void* gate;
  void* out; /* [T, H * vdim] */
  int64_t ldq, ldk, ldv, ldg, ldo;
  int32_t q_dtype, kv_dtype, gate_dtype, out_dtype;
  int32_t ntiles, H, dim, vdim;
  float scale;
} vila_sink_attn_params;
int vila_sink_attention(const vila_sink_attn_params* p, void* stream);

/* ---- blocks added for parallel-sublayer models with rotary grouped-query attention over a paged
 * K/V pool, short input convolutions, hashed token-pair embeddings and group-limited sigmoid routing.
 * Every mechanism is a parameterised call; nothing here is tied to one architecture. ------------- */

/* vila_glinear epilogue (flags): the weight rows are interleaved (gate_0, up_0, gate_1, ...) as for
 * VILA_FLAG_SWIGLU, out has N / 2 columns, and
 *   g = min(z_gate, act_limit), u = clamp(z_up, -act_limit, act_limit), out = g * sigmoid(act_alpha * g) * (u + 1)
 * act_alpha / act_limit travel in vila_glinear_ext, passed through vila_glinear_x. */
#define VILA_FLAG_GLU_CLAMP 4
/* act = VILA_ACT_XIELU: z > 0: act_pos z^2 + z / 2;  z <= 0: act_neg (e^z - 1 - z) + z / 2
 * in_scale (fp32, may be NULL; o_rows must be NULL then): the accumulators of sorted position i are
 *   multiplied by in_scale[a_rows ? a_rows[i] : i] BEFORE bias and activation, which is the layer applied
 *   to the scaled input row (a routing weight on an expert's input rather than on its output). */
#define VILA_ACT_XIELU 5
typedef struct vila_glinear_ext {
  float act_alpha, act_limit;
  float act_pos, act_neg;
  const float* in_scale;
} vila_glinear_ext;
int vila_glinear_x(const vila_glinear_params* p, const vila_glinear_ext* x, void* stream);

/* out[t, :] = table[ids[t], :] + pair_table[r(t), :] (fp32), with
 *   r(t) = prev_ids[t] < 0 ? buckets : (prev_ids[t] * mul_prev + ids[t] * mul_cur) mod buckets
 * (pair_table has buckets + 1 rows; the last one serves tokens without a predecessor). */
int vila_embed_pair_rows(const void* table, int table_dtype, const void* pair_table, int pair_dtype,
                         const int32_t* ids, const int32_t* prev_ids, int64_t mul_prev, int64_t mul_cur,
                         int64_t buckets, float* out, int rows, int cols, void* stream);

/* x[r, :] += vec  (fp32 stream, vec of any dtype) */
int vila_add_row_vector(float* x, const void* vec, int vec_dtype, int rows, int cols, void* stream);

/* RMS norm in `groups` equal consecutive pieces of every row, each with its own root mean square:
 *   out[r, c] = x[r, c] / sqrt(mean_{c' in piece(c)} x[r, c']^2 + eps) * (w[c] + w_offset) */
int vila_group_rmsnorm_rows(const void* x, int x_dtype, int64_t ldx, const void* w, int w_dtype,
                            float w_offset, float eps, void* out, int out_dtype, int64_t ldo, int rows,
                            int cols, int groups, void* stream);

/* Causal short convolution over time on every channel of ragged rows, with the input added back:
 *   out[t, c] = h[t, c] + sum_{j < taps} w[c, j] * h[t - (taps - 1) + j, c]
 * where rows before a sequence's portion come from its state slot (the last taps - 1 inputs of the
 * sequence, fp32 [slots, taps - 1, cols], oldest first) and rows before position 0 are zero.
 * row_seq[t] names the sequence of row t in seqs [nseq, 4] = (first row, rows, first position, slot).
 * vila_short_conv_state then stores the last taps - 1 inputs of every sequence (call it after the
 * convolution of the same step: it overwrites what the convolution reads). */
int vila_short_conv_rows(const float* h, const void* w, int w_dtype, const float* state,
                         const int32_t* seqs, const int32_t* row_seq, void* out, int out_dtype,
                         int rows, int cols, int taps, void* stream);
int vila_short_conv_state(const float* h, float* state, const int32_t* seqs, int nseq, int cols, int taps,
                          void* stream);

/* Rotary positions + unit norm + cache append for grouped-query attention.  qkv [T, ldq] holds q (H
 * heads of dim) | k (G heads of dim) | v (G heads of vdim).  On the first rot_dims columns of every q
 * and k head the pairs (2i, 2i+1) turn by positions[t] * inv_freq[i] (inv_freq fp64 [rot_dims / 2]);
 * then, if unit_norm, every q and k head is divided by sqrt(mean(head^2) + eps) and, where given,
 * multiplied by q_norm_w / k_norm_w (fp32 [dim], the same for every head).
 *   q_out fp32 [T, H * dim];  pool row cache_rows[t] = k (G * dim) | v (G * vdim) in pool_dtype.
 * v_from_k != 0: the row holds q | k only and the values are the keys as they came in (before rotation
 * and norm); vdim must equal dim. */
typedef struct vila_rope_append_params {
  const void* qkv;
  int64_t ldq;
  const int32_t* positions;
  const int32_t* cache_rows;
  const double* inv_freq;
  float* q_out;
  void* pool;
  int32_t qkv_dtype, pool_dtype, T, H, G, dim, vdim, rot_dims, unit_norm;
  float eps;
  const float* q_norm_w; /* [dim] or NULL */
  const float* k_norm_w; /* [dim] or NULL */
  int32_t v_from_k;
  int32_t rot_layout; /* 0: pairs (2i, 2i+1); 1: pairs (i, i + rot_dims / 2) */
  float rot_mscale;   /* cos and sin are multiplied by this; 0 counts as 1 */
} vila_rope_append_params;
int vila_rope_append(const vila_rope_append_params* p, void* stream);

/* vila_paged_attention — causal grouped-query attention over a paged pool whose rows are
 * k (G * dim) | v (G * vdim) per token, fp32 scores / softmax / weighted sum:
 *   s_h(i, j) = scale * <q_h(i), k_{h / (H / G)}(j)>;  if talk: s_h <- sum_g talk[h, g] s_g (all H heads
 *   of a (query, key) pair are mixed before the softmax);  j <= pos(i)
 *   if dist_bias: s_h += dist_bias[min(pos(i) - j, dist_rows - 1), h]   (after scale and mixing)
 *   if chunk > 0: only keys with floor(j / chunk) == floor(pos(i) / chunk) are seen (positions count
 *   from the start of the sequence, whatever the portion)
 *   p_h(i, j) = exp(s_h) / (sum_j exp(s_h) + exp(sink[h]))      (sink == NULL: ordinary softmax)
 *   out_h(i) = sum_j p_h(i, j) v_{h / (H / G)}(j);  if gate: out_h(i) *= sigmoid(gate[i, h])
 * tiles [ntiles, 4] = (first batch row, rows (<= 16), position of the first row, slot); page tables as
 * in vila_latent_attention.  nsplit > 1 (tiles of ONE row only: decoded tokens) deals the key blocks of
 * a row to nsplit CTAs; partial is fp32 [T, nsplit, H, vdim + 2], caller-owned. */
typedef struct vila_paged_attn_params {
  const float* q; /* [T, H * dim] */
  const void* pool;
  const int32_t* page_tables;
  const int32_t* tiles;
  const float* talk; /* [H, H] or NULL */
  const float* sink; /* [H] or NULL */
  void* out;         /* [T, H * vdim] */
  float* partial;
  int32_t pool_dtype, out_dtype, ntiles, pt_stride, H, G, dim, vdim, page, nsplit;
  int32_t max_rows; /* largest row count of any tile (1: decoded tokens only) */
  float scale;
  const float* dist_bias; /* [dist_rows, H] or NULL */
  const void* gate;       /* [T, ldg] pre-activations, column h = head h, or NULL */
  int64_t ldg;
  int32_t dist_rows, chunk, gate_dtype;
  /* window > 0: a key is seen only if pos(i) - j < window or j < keep_first (the first keep_first tokens
   * of a sequence stay visible, at their true positions); window == 0: no such limit.
   * talk_after != 0: talk mixes the heads' softmax WEIGHTS instead of their scores,
   *   p_h(i, j) <- sum_g talk[h, g] p_g(i, j), head h then sums the values of its own K/V head; the
   *   kernel makes two passes over the keys (running max and sum of every head first); no sink then.
   * head_scale fp32 [H] or NULL: the scores of head h are multiplied by head_scale[h] (before mixing). */
  int32_t window, keep_first, talk_after;
  const float* head_scale;
} vila_paged_attn_params;
int vila_paged_attention(const vila_paged_attn_params* p, void* stream);

/* Router with sigmoid scores and group-limited choice: s = sigmoid(w_router x) (fp32), choice = s +
 * correction; the experts form `groups` equal groups of neighbours, a group's score is the sum of its
 * two largest choice values (its only one if groups == experts), only experts of the `keep` best groups
 * can be chosen; the `top` largest choice values win (ties: the lower index); weight = s of the chosen
 * (not renormalised).  correction may be NULL.  idx / weight are [rows, top]. */
int vila_moe_route_sigmoid(const void* x, int x_dtype, int64_t ldx, const float* w_router,
                           const float* correction, int32_t* idx, float* weight, int rows, int cols,
                           int experts, int top, int groups, int keep, void* stream);

/* x[r, :] += mult * (a[r, :] + sum_{j < n_partials} part[r * n_partials + j, :])  (a or part may be NULL);
 * copy != NULL also receives the updated rows in copy_dtype (the next projection's operand). */
int vila_residual_add_rows(float* x, const void* a, int a_dtype, int64_t lda, const void* part,
                           int part_dtype, int64_t ldp, int n_partials, float mult, void* copy,
                           int copy_dtype, int rows, int cols, void* stream);

/* Pre-norm residual step in one pass: x[r, :] += a[r, :] + sum_{j < n_partials} part[r * n_partials + j, :] (a or
 * part may be NULL), then out[r, :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * w (w may be NULL): the updated stream
 * and the normed operand of the next sublayer.  out is [rows, cols] contiguous in out_dtype. */
int vila_residual_norm_rows(float* x, const void* a, int a_dtype, int64_t lda, const void* part, int part_dtype,
                            int64_t ldp, int n_partials, const void* w, int w_dtype, float eps, void* out,
                            int out_dtype, int rows, int cols, void* stream);

/* Group RMS norm + causal short convolution for up to two sublayers that read the same rows x, in one
 * pass (vila_group_rmsnorm_rows followed by vila_short_conv_rows / vila_short_conv_state per sublayer):
 *   h_k = groupnorm(x) * (norm_w[k] + w_offset);  out[k] = h_k + conv(h_k, conv_w[k]);  state[k] <- last inputs
 * The normalisation is shared, weights / taps / state / output are per sublayer (nsub = 1 or 2). */
typedef struct vila_norm_conv_params {
  const float* x; /* [rows, cols] contiguous */
  const float* norm_w[2];
  const void* conv_w[2]; /* [cols, taps] */
  float* state[2];       /* [slots, taps - 1, cols] */
  void* out[2];          /* [rows, cols] */
  const int32_t* seqs;
  const int32_t* row_seq;
  float* inv; /* scratch [rows, groups] (inverse root mean squares), or NULL: every CTA computes what it needs */
  int32_t conv_w_dtype, out_dtype, rows, nseq, cols, groups, taps, nsub;
  float eps, w_offset;
} vila_norm_conv_params;
int vila_norm_conv_rows(const vila_norm_conv_params* p, void* stream);

/* vila_gated_norm_residual with the update multiplied by `mult` */
int vila_gated_norm_residual_scaled(float* x, const void* part, int part_dtype, int64_t ldp, int n_partials,
                                    const void* gate, int gate_dtype, int64_t ldg, const void* gate_bias,
                                    int bias_dtype, const void* w, int w_dtype, float w_offset, float eps,
                                    float mult, int rows, int cols, void* stream);

/* out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j]   (z [T, cols] contiguous; a per-token side
 * input gated by a projection of the stream) */
int vila_gelu_mul_gather(const void* z, int z_dtype, const void* table, int table_dtype, int64_t ld_table,
                         const int32_t* ids, int col0, void* out, int out_dtype, int rows, int cols,
                         void* stream);

/* ---- State-space mixers on ragged batches: sinusoidal position embedding, causal depthwise
 * convolution with bias / SiLU, the scalar-decay (state-space duality) and the per-channel selective
 * recurrences, and the post-normed residual update of two scaled branches. ------------------------- */

/* out[t, c] = table[ids[t], c] * scale + (c odd ? cos : sin)(positions[t] * inv_freq[c / 2])
 * inv_freq fp64 [(cols + 1) / 2]; the angle is formed and reduced to [-pi, pi] in double.  copy (may be NULL)
 * also receives the rows in copy_dtype. */
int vila_embed_sincos_rows(const void* table, int table_dtype, const int32_t* ids, const int32_t* positions,
                           const double* inv_freq, float scale, float* out, void* copy, int copy_dtype,
                           int rows, int cols, void* stream);

/* x[r, :] += rms(sa * a[r, :] + sb * b[r, :]) * w   with rms(v) = v / sqrt(mean(v^2) + eps); b may be NULL.
 * copy (may be NULL) receives the updated rows in copy_dtype (the operand of the next projection). */
int vila_branch_norm_residual(float* x, const void* a, int a_dtype, int64_t lda, float sa, const void* b,
                              int b_dtype, int64_t ldb, float sb, const void* w, int w_dtype, float eps,
                              void* copy, int copy_dtype, int rows, int cols, void* stream);

#define VILA_CONV_SILU 1
/* Causal depthwise convolution over time on `cols` channels of ragged rows:
 *   out[t, c] = act(bias[c] + sum_{j < taps} w[c, j] * in[t - (taps - 1) + j, c])       (fp32 arithmetic)
 * Rows before a sequence's portion come from its state slot (fp32 [slots, taps - 1, cols], oldest first),
 * rows before position 0 are zero.  vila_causal_conv_state stores the last taps - 1 inputs of every
 * sequence afterwards (same params). */
typedef struct vila_causal_conv_params {
  const void* in; /* [rows, ld_in], the channels start at `in` */
  int64_t ld_in;
  const void* w;    /* [cols, taps] */
  const void* bias; /* [cols] or NULL, same dtype as w */
  float* state;
  const int32_t* seqs;    /* [nseq, 4] = (first row, rows, first position, slot) */
  const int32_t* row_seq; /* [rows] */
  void* out;
  int64_t ld_out;
  int32_t in_dtype, w_dtype, out_dtype, rows, nseq, cols, taps, act;
} vila_causal_conv_params;
int vila_causal_conv_rows(const vila_causal_conv_params* p, void* stream);
int vila_causal_conv_state(const vila_causal_conv_params* p, void* stream);

/* vila_ssd_scan — recurrence with one decay per head (state-space duality form), fp32 state:
 *   dt_t = softplus(dt_raw_t + dt_bias_h),  S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T,
 *   y_t = S_t^T C_t + D_h x_t,  out_t = y_t * silu(z_t) (z may be NULL)
 * xbc rows hold x (H heads of P) | B (G groups of N) | C (G groups of N); head h uses group h / (H / G).
 * state [slots, H, P, N] (N fastest); a sequence at position 0 starts from zero. */
typedef struct vila_ssd_scan_params {
  const void* xbc;
  int64_t ld_xbc;
  const void* dt; /* [rows, ld_dt], column h */
  int64_t ld_dt;
  const void* z; /* [rows, ld_z], H * P columns, or NULL */
  int64_t ld_z;
  const float* dt_bias; /* [H] */
  const float* A_log;   /* [H] */
  const float* D;       /* [H] */
  float* state;
  const int32_t* seqs;
  void* out; /* [rows, ld_out] */
  int64_t ld_out;
  int32_t in_dtype, out_dtype, nseq, H, P, N, G;
} vila_ssd_scan_params;
int vila_ssd_scan(const vila_ssd_scan_params* p, void* stream);

/* vila_selective_scan — recurrence with a step size and decay per channel, fp32 state [slots, C, N]:
 *   dt_t,c = softplus(dt_raw_t,c + dt_bias_c),  S_t[c, n] = exp(-exp(A_log[c, n]) dt_t,c) S_{t-1}[c, n] + dt_t,c x_t,c B_t,n
 *   y_t,c = sum_n S_t[c, n] C_t,n + D_c x_t,c,  out = y * silu(z) (z may be NULL)
 * bc rows hold B (N) | C (N). */
typedef struct vila_selective_scan_params {
  const void* x; /* [rows, ld_x] */
  int64_t ld_x;
  const void* dt; /* [rows, ld_dt] */
  int64_t ld_dt;
  const void* bc;
  int64_t ld_bc;
  const void* z;
  int64_t ld_z;
  const float* dt_bias; /* [C] */
  const float* A_log;   /* [C, N] */
  const float* D;       /* [C] */
  float* state;
  const int32_t* seqs;
  void* out;
  int64_t ld_out;
  int32_t in_dtype, out_dtype, nseq, C, N;
} vila_selective_scan_params;
int vila_selective_scan(const vila_selective_scan_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VILA_B200_H_ */
