/* pg_b200 — C ABI of the B200-native PaliGemma hot path.
 *
 * The reference (PhilipWilliamVentura/multimodal-financial-analysis-tool-using-paligemma)
 * is pure Python/PyTorch and has no FFI of its own: its boundary is the
 * Python class surface of modeling_gemma.py / modeling_siglip.py.  Our drop-in modules of
 * the same names call these entry points (ctypes); every entry names
 * the reference code it replaces.
 *
 * Conventions: plain device pointers and sizes, no torch types; `stream` is a
 * cudaStream_t passed as void*; every call is asynchronous on that stream, allocates
 * nothing and never synchronises; return 0 on success, non-zero otherwise with a message
 * in pg_last_error().  `dtype` selects the model dtype of activations and weights
 * (PG_F32 is the fp32 verification mode: true fp32 FMA, no TF32).  Matrices are row-major;
 * weights are [out_features, in_features] exactly as torch.nn.Linear stores them.
 */
#ifndef PG_B200_H
#define PG_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { PG_F32 = 0, PG_BF16 = 1, PG_F16 = 2 };
enum { PG_OK = 0, PG_ERR_INVALID = 1, PG_ERR_CUDA = 2 };

/* pg_gemm epilogues (all round to the model dtype where the reference materialises a tensor) */
enum {
  PG_EPI_NONE = 0,      /* C = A W^T                                  */
  PG_EPI_BIAS = 1,      /* C = A W^T + b                  nn.Linear   */
  PG_EPI_BIAS_GELU = 2, /* C = gelu_tanh(A W^T + b)       SiglipMLP fc1 */
  PG_EPI_BIAS_RES = 3,  /* C = (A W^T + b) + R            out_proj / fc2 / patch-embed+pos */
  PG_EPI_RES = 4,       /* C = (A W^T) + R                o_proj / down_proj */
  PG_EPI_GEGLU = 5,     /* C = gelu_tanh(A Wg^T) * (A Wu^T), W = [Wg; Wu]  GemmaMLP */
  PG_EPI_SWIGLU = 6     /* C = silu(A Wg^T) * (A Wu^T), W = [Wg; Wu]       gated experts */
};

/* One exchange of the tensor-parallel decoder over NVLink peer memory (csrc/tp_exchange.cuh; SURVEY.md §8e: the
 * reference is single-device, the sharding is the north star's).  The PRODUCER kernel stores this rank's fp32 partial
 * as {value, sequence number} words into slot (parity, rank) of EVERY rank's buffer; the CONSUMER kernel waits for all
 * `size` slots of its local buffer and sums them in rank order.  Passed by pointer (host memory, read at launch);
 * NULL means "not tensor parallel" everywhere a parameter of this type appears. */
typedef struct pg_tp_exchange {
  const void* peers;    /* device array of `size` pointers: base address of every rank's exchange buffer        */
  const int* epoch;     /* device int: decode-step counter of this rank, advanced by pg_tp_begin_step           */
  int* err_dev;         /* device int: set when a wait timed out (lost peer); later waits return at once         */
  int* err_host;        /* pinned host int mirrored from err_dev (may be NULL)                                   */
  long long region_off; /* byte offset of this exchange's region inside the buffers                              */
  long long slot_bytes; /* bytes of one (parity, source rank) slot: 8 per fp32 word                              */
  int rank, size;       /* this rank, number of ranks (2..8)                                                     */
  int index, stride;    /* sequence number = *epoch * stride + index, 1 <= index < stride; exchanges that follow  */
                        /* one another in the same region must alternate the parity of `index`                   */
} pg_tp_exchange;

const char* pg_last_error(void);
int pg_abi_version(void);
/* number of kernels this library has launched since load (bench.py's gpu_launches) */
unsigned long long pg_launch_count(void);

/* ---- embedding + image/text merge + sqrt(D) normaliser --------------------------------
 * Replaces nn.Embedding lookup (modeling_gemma.py:565), _merge_input_ids_with_image_features
 * (:476-500) and the `hidden_states * normalizer` of GemmaModel.forward (:367-368).
 * out[t] = 0 for pad ids; rnd(rnd(img[k]/img_div) * normalizer) for the k-th image token in
 * row-major order; rnd(emb[id] * normalizer) otherwise.  ids may be int64 device memory.
 * If an image token has no image row left (reference: masked_scatter raises) or an id is out
 * of range, *err_flag (device int, may be NULL) is set to 1 and the row is zero. */
int pg_embed_merge(void* out, const int64_t* ids, const void* emb, const void* img_feats,
                   int n_tokens, int D, int64_t vocab, int64_t image_token_id, int64_t pad_id,
                   int n_img_rows, float img_div, float normalizer, int* err_flag,
                   int dtype, void* stream);

/* GemmaRMSNorm.forward (modeling_gemma.py:114-120) */
int pg_rmsnorm(void* out, const void* x, const void* w, int rows, int D, float eps,
               int dtype, void* stream);
/* nn.LayerNorm (modeling_siglip.py:175,177,234) */
int pg_layernorm(void* out, const void* x, const void* w, const void* b, int rows, int D,
                 float eps, int dtype, void* stream);

/* Image pre-processing on the device (processing_paligemma.py:13-50).  pg_resample_u8 is one pass of Pillow's 8-bit
 * bicubic resize (Image.resize(..., BICUBIC), libImaging/Resample.c) along one axis of an interleaved uint8 image:
 * vertical == 0: in (rows, n_in, C) -> out (rows, n_out, C); vertical != 0: in (n_in, rows, C) -> out (n_out, rows, C).
 * bounds int32 [n_out][2] = (first input index, tap count), kk int32 [n_out][ksize] = 22-bit fixed-point taps, both
 * from the host (pg_b200/preprocess.py::resample_coeffs).  Horizontal pass first, then vertical, as Pillow does.
 * pg_u8_to_chw: out[c][y][x] = lut[in[y][x][c]] in the model dtype; lut float32 [256] = ((b/255) - mean) / std with
 * the reference's dtypes (pg_b200/preprocess.py::value_table). */
int pg_resample_u8(uint8_t* out, const uint8_t* in, const int32_t* bounds, const int32_t* kk, int ksize,
                   int rows, int n_in, int n_out, int channels, int vertical, void* stream);
int pg_u8_to_chw(void* out, const uint8_t* in, const float* lut, int H, int W, int channels, int dtype,
                 void* stream);

/* SiglipVisionEmbeddings patch conv as im2col (modeling_siglip.py:45-51,67-73): stride == kernel
 * so it is a pure permutation: out[(b*P + py*G + px), c*p*p + ky*p + kx], row stride ld_out
 * (columns beyond C*p*p are zero-filled up to ld_out). */
int pg_im2col(void* out, const void* pixels, int B, int C, int H, int W, int p, int ld_out,
              int dtype, void* stream);

/* C[M,N] = A[M,K] W[N,K]^T with a fused epilogue; fp32 accumulation.  R row index is
 * m % res_mod when res_mod > 0 (position-embedding broadcast over the batch).  out_f32 != 0
 * stores fp32 (lm_head `.float()`, modeling_gemma.py:417-418).  impl: 0 = auto, 1 = SIMT
 * (any dtype), 2 = tcgen05/TMA (bf16/f16 only; picks the CTA-pair, single-CTA, skinny or split-K kernel by shape),
 * 3 = the CTA-pair swap-AB kernel for 129..512 rows (weights as the M operand, split-K through pg_set_workspace;
 * auto takes it for the projections where it measured faster).  Replaces every nn.Linear / matmul call site
 * of SURVEY.md §2.3 on the prefill and vision paths. */
int pg_gemm(void* C, const void* A, const void* W, const void* bias, const void* R,
            int M, int N, int K, int lda, int ldw, int ldc, int ldr, int res_mod,
            int epilogue, int out_f32, int impl, int dtype, void* stream);

/* Scratch memory for GEMMs that split K over CTA pairs (prompt-sized row counts: csrc/gemm_tcgen05_swap.cu): a
 * caller-owned device buffer the library may overwrite during any pg_gemm call on this device (fp32 partials
 * [splits][M][N]); without one (or with one that is too small for a problem) pg_gemm takes its other kernels.
 * The library never allocates. */
int pg_set_workspace(void* ptr, long long bytes);

/* RoPE on q and k + append of K,V to the paged cache (modeling_gemma.py:155-199, 23-36).
 * qkv: [B*q_len, (nq+2*nkv)*hd] from the fused projection; q_out: [B*q_len, nq*hd].
 * Token (b,i) gets position positions[b*q_len+i] (clamped to [0,max_pos-1]) and cache slot
 * slot_base[b]+i.  Pools are [num_pages, page_size, nkv*hd]. */
int pg_rope_append(void* q_out, const void* qkv, const float* inv_freq, const int32_t* positions,
                   void* k_pool, void* v_pool, const int32_t* page_table, int pt_stride,
                   int page_size, const int32_t* slot_base, int B, int q_len, int nq, int nkv,
                   int hd, int max_pos, int dtype, void* stream);

/* Unmasked softmax attention (the reference's additive mask is all zeros: modeling_gemma.py:
 * 506-514; SigLIP has none: modeling_siglip.py:116-131).  fp32 softmax.  q: [B*q_len, ld_q],
 * head h at column h*hd.  K/V either contiguous (page_table NULL: row (b,j) at
 * base + b*kv_batch_stride + j*ld_kv elements) or paged.  kv_len: device int32[B] or NULL
 * (then kv_len_const).  kv_len_add is added to the device value.  scale_mode 0: s*scale
 * (SigLIP), 1: s/scale (Gemma). */
int pg_attention(void* out, int ld_out, const void* q, int ld_q, const void* k, const void* v,
                 int ld_kv, long long kv_batch_stride, const int32_t* page_table, int pt_stride,
                 int page_size, const int32_t* kv_len, int kv_len_const, int kv_len_add, int B,
                 int q_len, int n_heads, int n_kv_heads, int hd, float scale, int scale_mode,
                 int dtype, void* stream);

/* The same attention on the tcgen05 tensor cores (16-bit dtypes; prefill, cache-off recompute, SigLIP):
 * QK^T and PV as tcgen05.mma with TMEM accumulators, Q/K/V tiles by TMA, two-pass softmax (row max, then
 * exp / PV) with one thread per query row.  q, k, v are row-major matrices (`*_rows` x `ld_*`); head h sits
 * at columns *_col0 + h*hd_stride .. +hd, and a head row must be padded (with zeros) to a multiple of 64
 * columns unless hd is 128 or 256.  Paged K/V needs page_size == key tile (128 for hd <= 128, 64 above).
 * Output is packed: head h at column h*hd of [B*q_len, ld_out]. */
int pg_attention_tc(void* out, int ld_out, const void* q, long long q_rows, int ld_q, int q_col0,
                    const void* k, const void* v, long long kv_rows, int ld_kv, int k_col0, int v_col0,
                    int hd_stride, long long kv_batch_rows, const int32_t* page_table, int pt_stride,
                    int page_size, const int32_t* kv_len, int kv_len_const, int kv_len_add, int B, int q_len,
                    int n_heads, int n_kv_heads, int hd, float scale, int scale_mode, int dtype, void* stream);

/* ---- decode path (q_len == 1 per sequence), B <= PG_MAX_DECODE_BATCH per call ----------- */
#define PG_MAX_DECODE_BATCH 8

/* L2 prefetch chain: registers [ptr, ptr+bytes) (16-byte aligned; normally the NEXT kernel's
 * weights) with the calling thread; the next pg_decode_* / pg_gemv_res launch from this thread
 * consumes it and starts by issuing cp.async.bulk.prefetch.L2 for that region, one slice per CTA.
 * Weights never depend on activations, so HBM keeps streaming through the small latency-bound
 * kernels and across kernel boundaries.  Purely a performance hint: results never change. */
int pg_set_next_prefetch(const void* ptr, long long bytes);

/* input RMSNorm + fused q/k/v projection + RoPE + KV append (GemmaDecoderLayer.forward
 * :314-316, GemmaAttention.forward :241-259).  x: [B,D] residual stream. positions/kv_len:
 * device int32[B]; K,V go to slot kv_len[b]. */
int pg_decode_qkv(void* q_out, const void* x, const void* norm_w, const void* w_qkv,
                  const float* inv_freq, const int32_t* positions, void* k_pool, void* v_pool,
                  const int32_t* page_table, int pt_stride, int page_size, const int32_t* kv_len,
                  int B, int D, int nq, int nkv, int hd, float eps, int max_pos,
                  const pg_tp_exchange* ex, void* x_out, int dtype, void* stream);
/* ex != NULL (tensor parallel; same meaning in pg_decode_gateup / pg_decode_lmhead): the residual stream this
 * kernel normalises is x_new = rnd(x + rnd(sum over ranks of the fp32 partials of exchange `ex`)), i.e. the
 * all-reduce of the previous o_proj / down_proj and the `residual + hidden_states` of modeling_gemma.py:327,336
 * happen in this kernel's prologue; x_new is also written to x_out [B,D] (must not alias x). */

/* split-K MQA attention over the paged cache for one new token per sequence
 * (modeling_gemma.py:262-288).  Attends kv_len[b]+kv_len_add entries.  ws: fp32 workspace of
 * pg_decode_attention_ws_floats() floats; counters: int32[B*nkv], zero before first use. */
long long pg_decode_attention_ws_floats(int B, int nq, int hd, int max_splits);
int pg_decode_attention(void* out, const void* q, const void* k_pool, const void* v_pool,
                        const int32_t* page_table, int pt_stride, int page_size,
                        const int32_t* kv_len, int kv_len_add, int B, int nq, int nkv, int hd,
                        float scale_div, float* ws, int* counters, int max_splits, int dtype,
                        void* stream);

/* out[B,N] = (x[B,K] W[N,K]^T) + R  — o_proj / down_proj with the residual add
 * (modeling_gemma.py:291,327 and :134,336).  R may be NULL.  ex != NULL (tensor parallel: W holds this rank's K
 * columns): the unrounded fp32 partial x W^T goes to word b*N+n of this rank's slot in every rank's exchange buffer
 * instead; out and R are ignored (the consumer adds the residual). */
int pg_gemv_res(void* out, const void* x, const void* W, const void* R, int B, int N, int K,
                const pg_tp_exchange* ex, int dtype, void* stream);

/* post-attention RMSNorm + gate/up projections + GeGLU (modeling_gemma.py:332,134).
 * w_gu = [Wgate; Wup] : [2F, D];  out: [B,F]. */
int pg_decode_gateup(void* out, const void* x, const void* norm_w, const void* w_gu, int B,
                     int D, int F, float eps, const pg_tp_exchange* ex, void* x_out, int dtype, void* stream);

/* final RMSNorm + tied lm_head + fp32 logits + greedy argmax (modeling_gemma.py:379,417-418;
 * inference.py:68).  logits: fp32 [B,V] (values rounded to the model dtype first, as the
 * reference's `.float()` of a model-dtype tensor).  argmax_keys: device u64[B], must hold 0
 * on entry; decoded by pg_step_advance.  Ties go to the lowest index. */
int pg_decode_lmhead(float* logits, const void* x, const void* norm_w, const void* w_emb,
                     int B, int D, int64_t V, float eps, unsigned long long* argmax_keys,
                     const pg_tp_exchange* ex, void* x_out, int dtype, void* stream);

/* End of a decode step, all on device (replaces the host side of inference.py:68-78):
 * token[b] = argmax(keys[b]) (or sampled[b] if sampled != NULL); next_ids[b] = token;
 * history[b*hist_stride + step_counter] = token; kv_len[b] += 1; positions[b] += 1;
 * keys[b] = 0; *step_counter += 1 (by thread 0). */
int pg_step_advance(int64_t* next_ids, int64_t* history, int hist_stride, int* step_counter,
                    unsigned long long* keys, const int64_t* sampled, int32_t* kv_len,
                    int32_t* positions, int B, const pg_tp_exchange* keys_ex, void* stream);
/* keys_ex != NULL (tensor parallel, greedy): token[b] is decoded from the largest key over the ranks' vocabulary
 * shards, waited for in the key exchange filled by pg_tp_keys_push (ties: lowest global index). */

/* Head of a cached decode step driven through the reference API (inference.py:56-63,
 * modeling_gemma.py:557-559): ids_dst[b] = ids_src[b]; positions[b] = position; and the reference's
 * "The input cannot be padded" check without a host synchronisation: *bad_flag (any device-visible int,
 * e.g. pinned host memory) is set to 1 when one of the mask_n attention-mask elements is not 1.
 * mask_kind: 0 int64, 1 float32, 2 int32, 3 bfloat16, 4 float16, 5 uint8/bool, 6 float64; mask may be NULL. */
int pg_decode_inputs(int64_t* ids_dst, const int64_t* ids_src, int32_t* positions, int position,
                     const void* mask, int mask_kind, long long mask_n, int* bad_flag, int B, void* stream);

/* torch.argmax(logits, -1) over fp32 [B,V] (inference.py:68).  keys_ws: device u64[B] holding 0
 * on entry (left 0 on exit).  out == NULL: stop after the packed (value, index) keys, which stay in keys_ws
 * (tensor parallel: the shard's keys go to pg_tp_keys_push). */
int pg_argmax(int64_t* out, const float* logits, unsigned long long* keys_ws, int B, int64_t V,
              void* stream);

/* softmax(logits/temperature) + nucleus (top-p) sampling (inference.py:15-24,65-66).
 * The nucleus is the reference's: descending order, keep while (cumsum - p_i) <= top_p;
 * the draw uses counter-based Philox (seed, *rng_offset + b) rather than torch's RNG stream.
 * probs_ws: fp32 [B,V] scratch. nucleus_size (int32[B], may be NULL) reports the kept count. */
int pg_top_p_sample(int64_t* out, const float* logits, float* probs_ws, int B, int64_t V,
                    float temperature, float top_p, unsigned long long seed,
                    const int* rng_offset, int* nucleus_size, void* stream);

/* ---- tensor-parallel decoder plumbing (pg_tp_exchange above) --------------------------------------------------
 * pg_tp_begin_step: *epoch += 1, once at the head of every decode step (before its first producer).
 * pg_tp_push: producer for a partial that a GEMM left in local memory (batched decode step): partial[n] fp32 ->
 *   words 0..n-1 of this rank's slot in every rank's buffer.
 * pg_rmsnorm_reduce: consumer for that step, one CTA per row: x_new = rnd(x_in + rnd(sum of partials)) -> x_out,
 *   out = GemmaRMSNorm(x_new) (modeling_gemma.py:114-120).  x_out must not alias x_in.
 * pg_tp_keys_push: vocabulary-split lm_head: keys[b] (value, LOCAL index) -> (value, index + rank * v_local) in
 *   every rank's key slot; pg_step_advance(keys_ex) picks the winner. */
int pg_tp_begin_step(int* epoch, void* stream);
int pg_tp_push(const float* partial, long long n, const pg_tp_exchange* ex, void* stream);
int pg_rmsnorm_reduce(void* out, void* x_out, const void* x_in, const void* w, int rows, int D, float eps,
                      const pg_tp_exchange* ex, int dtype, void* stream);
int pg_tp_keys_push(const unsigned long long* keys, int B, long long v_local, const pg_tp_exchange* ex,
                    void* stream);

/* KVCache.key_cache[layer] / value_cache[layer] view: gather pages into a contiguous
 * [B, nkv, T, hd] tensor (modeling_gemma.py:12-36 attribute parity). */
int pg_kv_gather(void* out, const void* pool, const int32_t* page_table, int pt_stride,
                 int page_size, int B, int T, int nkv, int hd, int dtype, void* stream);

/* ---- ragged token batches (decoder-only models behind the slot scheduler) -----------------------------------------
 * A step is a flat list of n_tokens tokens.  Token t belongs to the sequence whose pages are row tok_slot[t] of the
 * page table and sits at position tok_pos[t] of it, so portions of prompts and single decoded tokens of different
 * sequences share every launch.  The residual stream x is fp32 [n_tokens, D] whatever the model dtype. */

/* x[t] = emb[ids[t]] * emb_scale + pos_emb[positions[t]]  (pos_emb may be NULL).  A bad id or position sets *err_flag
 * and gives a zero row. */
int pg_embed_pos(float* x, const int64_t* ids, const int32_t* positions, const void* emb, const void* pos_emb,
                 int n_tokens, int D, int64_t vocab, int max_pos, float emb_scale, int* err_flag, int dtype,
                 void* stream);

/* Residual sum + RMS norm in groups.  x[r] += add_a[r] + add_b[r] (model dtype, either may be NULL; written back),
 * then every one of the `groups` equal consecutive parts of the row is divided by sqrt(mean(part^2) + eps) and the
 * row is multiplied by w: out (model dtype, packed rows).  out == NULL: only the sum.  rows_idx (device int32, may be
 * NULL, not together with a sum) picks the input rows.  groups == 1 is the ordinary RMS norm. */
int pg_group_rmsnorm(void* out, float* x, const void* add_a, int lda, const void* add_b, int ldb, const void* w,
                     const int32_t* rows_idx, int rows, int D, int groups, float eps, int dtype, void* stream);

/* RMS norm of the query row and of the key row over ALL their columns (q_w / k_w NULL: no norm), then the key and
 * value rows go to the paged pools ([pages, page_size, k_cols] and [.., v_cols]) at (tok_slot, tok_pos).  proj holds
 * the fused projection, row stride ld.  k_cols == 0: a layer that attends another layer's cache. */
int pg_qknorm_append(void* q_out, const void* proj, int ld, int q_col0, int q_cols, int k_col0, int k_cols,
                     int v_col0, int v_cols, const void* q_w, const void* k_w, float eps, void* k_pool, void* v_pool,
                     const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                     const int32_t* tok_pos, int n_tokens, int dtype, void* stream);

/* Causal attention of every token over its sequence's cache: keys j with 0 <= pos - j < window (window <= 0: all
 * j <= pos), score = (q . k_j) * scale - slopes[h] * (pos - j) (slopes: device float[n_heads] or NULL), fp32 softmax,
 * query head h reads key/value head h / (n_heads / n_kv_heads), key width dim, value width vdim; the result is
 * multiplied by sigmoid(gate) when gate != NULL (same layout as out) and rounded once.  ws (fp32 scratch of ws_floats
 * floats, may be NULL): decode-sized steps split the keys of a token over several CTAs and merge through it. */
int pg_attention_ragged(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                        const void* k_pool, const void* v_pool, const int32_t* page_table, int pt_stride,
                        int page_size, const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int n_heads,
                        int n_kv_heads, int dim, int vdim, float scale, int window, const float* slopes, float* ws,
                        long long ws_floats, int dtype, void* stream);

/* The same attention on the tcgen05 tensor cores for prompt portions (16-bit dtypes, dim and vdim multiples of 64 up
 * to 256, page_size 64; pg_attention_ragged_tc_ok tells).  `tiles` (device int32 [n_tiles][4]) cuts the step's tokens
 * into runs of up to 128 consecutive tokens of one sequence at consecutive positions: {first token row, rows,
 * page-table row, position of the first row}; every token of the step must lie in exactly one tile.  pool_rows =
 * pages * page_size.  Softmax weights are computed in fp32 and rounded to the model dtype as the operand of P V.
 * Its pipeline waits are bounded; *err_flag (device-visible int, may be NULL) becomes 2 if one gives up. */
int pg_attention_ragged_tc_ok(int dim, int vdim, int page_size, int ld_q, int ld_out, int ld_gate, int dtype);
int pg_attention_ragged_tc(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                           const void* k_pool, const void* v_pool, long long pool_rows, const int32_t* page_table,
                           int pt_stride, int page_size, const int32_t* tiles, int n_tiles, int n_tokens, int n_heads,
                           int n_kv_heads, int dim, int vdim, float scale, int window, const float* slopes,
                           int* err_flag, int dtype, void* stream);

/* The same with three extensions.  keep_first > 0: positions < keep_first of the sequence stay visible behind the
 * window (at their true positions).  sigmoid_weights != 0: no softmax; the weight of a visible key is
 * sigmoid(score + head_bias[h]) (head_bias: device float[n_heads] or NULL, also added under the softmax) and the
 * weights are not normalised.  gate_per_head != 0: gate holds one value per (token, head) at gate[t * ld_gate + h]
 * instead of one per output column.  The result is multiplied by out_scale before it is rounded. */
int pg_attention_ragged_ex(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                           int gate_per_head, const void* k_pool, const void* v_pool, const int32_t* page_table,
                           int pt_stride, int page_size, const int32_t* tok_slot, const int32_t* tok_pos,
                           int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, float scale, int window,
                           int keep_first, const float* slopes, int sigmoid_weights, const float* head_bias,
                           float out_scale, float* ws, long long ws_floats, int dtype, void* stream);

/* pg_attention_ragged_tc with the extensions of pg_attention_ragged_ex (kept first positions, sigmoid weights with a
 * per-head bias in ONE pass over the key tiles, per-head gate, out_scale). */
int pg_attention_ragged_tc_ex(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                              int gate_per_head, const void* k_pool, const void* v_pool, long long pool_rows,
                              const int32_t* page_table, int pt_stride, int page_size, const int32_t* tiles,
                              int n_tiles, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, float scale,
                              int window, int keep_first, const float* slopes, int sigmoid_weights,
                              const float* head_bias, float out_scale, int* err_flag, int dtype, void* stream);

/* Bias, rotary positions, value mixing and cache append for one fused projection row per token: proj row holds
 * n_heads query heads and n_kv_heads key heads of `dim` columns and n_kv_heads value heads of `vdim` columns at the
 * given offsets.  Biases (model dtype, may be NULL) are added first.  The first rot_dims columns of every query and
 * key head are rotated in pairs ((2i, 2i+1) when interleaved != 0, else (i, i + rot_dims/2)) by the angle
 * position * freq[i] (freq: device float[rot_dims / 2]), cos and sin both multiplied by mag; fp32 angles.  v_first != NULL: the value row
 * becomes (1 - lambda) v + lambda v_first[t] (row stride ld_vf) before it is cached.  Queries go to q_out (packed),
 * keys and values to the paged pools at (tok_slot, tok_pos). */
int pg_rotary_append(void* q_out, const void* proj, int ld, int q_col0, int n_heads, int k_col0, int n_kv_heads,
                     int dim, int v_col0, int vdim, const void* q_bias, const void* k_bias, const void* v_bias,
                     const float* freq, int rot_dims, float mag, int interleaved, const void* v_first, int ld_vf,
                     float lambda, void* k_pool, void* v_pool, const int32_t* page_table, int pt_stride,
                     int page_size, const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int dtype,
                     void* stream);

/* Output norm of a sublayer + layer scale + residual sum + the next input norm:
 * x[r] += scale (.) (y[r] / sqrt(mean(y[r]^2) + eps) * w_post)   (scale: per channel, may be NULL);
 * out != NULL: out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w_next (model dtype, packed).  x is the fp32 stream. */
int pg_postnorm_residual(void* out, float* x, const void* y, int ldy, const void* w_post, const void* scale,
                         const void* w_next, int rows, int D, float eps, int dtype, void* stream);

/* ---- recurrent mixers: generalised delta rule ---------------------------------------------------------------------
 * Per head, state S [dim x dim] in fp32 per sequence slot ([slots][heads][dim][dim]):
 *   u = k / sqrt(sum(k^2) + key_eps);  S <- diag(w) S - (a * u)(u^T S) + k v^T;  o = S^T r.
 * pg_delta_prep: from the fused projection row (r, k, v, the removal gate's pre-activation a and the decay's inner
 *   projection of width `lora` at their column offsets) one packed fp32 record per (token, head):
 *   [r | k | w | u | a*u | v], each dp = dim rounded up to 4 floats (padding zero), with
 *   w = exp(-decay_scale * sigmoid(W2 tanh(inner) + w0)) (W2 [heads * dim, lora], product in fp32) and
 *   a = sigmoid(a + a_bias).  rec holds pg_delta_record_floats(n_tokens, heads, dim) floats.
 * pg_delta_rule: segs (device int32 [n_segs][3] = {state slot, first token row, tokens}; consecutive rows of one
 *   sequence in order; 0 tokens: skipped) are advanced from the slot's state, which is updated in place;
 *   out fp32 [n_tokens, heads * dim].
 * pg_headnorm_gate: out[t, h*dim + c] = o / sqrt(mean_h(o^2) + eps) * w[h*dim + c] * sigmoid(gate[t, h*dim + c]) *
 *   out_scale, rounded to the model dtype (w, gate may be NULL). */
long long pg_delta_record_floats(int n_tokens, int heads, int dim);
int pg_delta_prep(float* rec, const void* proj, int ld, int r_col0, int k_col0, int v_col0, int a_col0, int lora_col0,
                  int lora, const void* w2, const void* w0, const void* a_bias, int n_tokens, int heads, int dim,
                  float decay_scale, float key_eps, int dtype, void* stream);
int pg_delta_rule(float* out, float* state, const float* rec, const int32_t* segs, int n_segs, int heads, int dim,
                  void* stream);
int pg_headnorm_gate(void* out, int ld_out, const float* o, const void* w, const void* gate, int ld_gate, int n_tokens,
                     int heads, int dim, float eps, float out_scale, int dtype, void* stream);

/* xIELU: z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2;  (p, q) = pq[0..1] in
 * the model dtype.  out may alias z. */
int pg_xielu(void* out, const void* z, const void* pq, long long n, int dtype, void* stream);

/* out[r, c] = silu(gate_up[r, c]) * gate_up[r, F + c] for a [rows, 2F] matrix (model dtype): the pairing of a stacked
 * gate/up projection that was computed without it (the weight-streaming kernels of decode-sized steps). */
int pg_swiglu(void* out, const void* gate_up, int rows, int F, int dtype, void* stream);
/* The same pairing with the tanh form of GELU on the gate: out = gelu_tanh(gate) * up. */
int pg_geglu(void* out, const void* gate_up, int rows, int F, int dtype, void* stream);

/* ---- mixture of experts ---------------------------------------------------------------------------------------
 * pg_moe_route: z = h W_router^T in fp32, s = softmax(z) over all n_route outputs, the `top` largest of
 *   s + correction are chosen (ties: lowest index), topk_w = s * scale (not renormalised).  w_shared_gate != NULL:
 *   shared_gate[t] = sigmoid(h . w_shared_gate).
 * pg_moe_sort: the n_pairs = n_tokens * top pairs with index < n_experts are grouped by expert: offsets[n_experts+1],
 *   sorted_row[pos] = token row of the pair at sorted position pos, pair_pos[pair] = its position or -1 (an index
 *   >= n_experts is an identity expert: its output is the token's own input).
 * pg_moe_gemm: out[pos] = A[row_map ? row_map[pos] : pos] W_e^T for offsets[e] <= pos < offsets[e+1]; W is
 *   [n_experts][N (2N with swiglu)][K]; swiglu: silu(A Wg^T) * (A Wu^T) with W_e = [Wg; Wu].  impl 0 auto, 1 fp32
 *   FMA kernel, 2 tcgen05 kernel (16-bit dtypes, rows already grouped: row_map NULL; its pipeline waits are bounded and
 *   *err_flag, a device-visible int that may be NULL, becomes 2 if one gives up).
 * pg_moe_combine: x[t] += sum_k topk_w[t,k] * (y[pair_pos[t,k]] or h[t]) + shared_gate[t] * shared_out[t]. */
int pg_moe_route(int32_t* topk_idx, float* topk_w, float* shared_gate, const void* h, int ldh, const void* w_router,
                 const void* correction, const void* w_shared_gate, int n_tokens, int D, int n_route, int top,
                 float scale, int dtype, void* stream);
int pg_moe_sort(int32_t* offsets, int32_t* sorted_row, int32_t* pair_pos, const int32_t* topk_idx, int n_pairs,
                int top, int n_experts, void* stream);
int pg_moe_gemm(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int swiglu, int impl, int* err_flag,
                int dtype, void* stream);
/* out[r] = a[row_map[r]] for r < *n_rows (n_rows: device int, NULL = all max_rows): packed rows of `cols` elements. */
int pg_gather_rows(void* out, const void* a, int lda, const int32_t* row_map, const int32_t* n_rows, int max_rows,
                   int cols, int dtype, void* stream);
int pg_moe_combine(float* x, const void* y, int ldy, const int32_t* pair_pos, const float* topk_w, const void* h,
                   int ldh, const void* shared_out, int lds, const float* shared_gate, int n_tokens, int D, int top,
                   int dtype, void* stream);

/* pairings of the two products of a stacked [Wg; Wu] weight (pg_moe_gemm_act, pg_glu_clamped) */
enum {
  PG_GLU_NONE = 0,
  PG_GLU_SILU = 1,    /* silu(g) * u */
  PG_GLU_CLAMPED = 2  /* g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1) */
};

/* pg_moe_gemm with the pairing given by name (pg_moe_gemm: swiglu != 0 is PG_GLU_SILU). */
int pg_moe_gemm_act(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                    const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int act, float limit, int impl,
                    int* err_flag, int dtype, void* stream);
/* Router with sigmoid scores and expert groups: z = h W_router^T in fp32, s = sigmoid(z), choice c = s + correction
 * (correction may be NULL).  The n_route experts form n_groups equal groups of neighbours; a group's score is the sum
 * of its two largest choice scores, only experts of the `keep` best groups can be chosen; the `top` largest choice
 * scores are chosen (ties: lowest index) and topk_w = s[chosen] / (sum of the chosen s + 1e-20). */
int pg_moe_route_grouped(int32_t* topk_idx, float* topk_w, const void* h, int ldh, const void* w_router,
                         const void* correction, int n_tokens, int D, int n_route, int top, int n_groups, int keep,
                         int dtype, void* stream);
/* out[t] = sum_k topk_w[t,k] * y[pair_pos[t,k]] + shared_out[t] (shared_out may be NULL), rounded to the model dtype:
 * the feed-forward output of designs that norm it before the residual sum. */
int pg_moe_combine_out(void* out, int ldo, const void* y, int ldy, const int32_t* pair_pos, const float* topk_w,
                       const void* shared_out, int lds, int n_tokens, int D, int top, int dtype, void* stream);
/* out[r, c] = g sigmoid(alpha g) (u + 1), g = min(gate_up[r, c], limit), u = clamp(gate_up[r, F + c], -limit, limit). */
int pg_glu_clamped(void* out, const void* gate_up, int rows, int F, float limit, float alpha, int dtype, void* stream);

/* ---- lightning attention: linear attention with a constant decay per head ------------------------------------------
 * Per head, state S [dim x vdim] in fp32 per sequence slot ([slots][heads][dim][vdim]); q, k, v = silu of the fused
 * projection's columns at q_col0 / k_col0 / v_col0 (heads x dim, heads x dim, heads x vdim):
 *   S <- decay[h] S + k v^T;  o = S^T q.   segs as for pg_delta_rule; out fp32 [n_tokens, heads * vdim].
 * pg_lightning_prep writes rec: pg_lightning_record_floats(n_tokens, heads, dim, vdim) floats (the fp32 activations,
 * one packed record [q | k | v] per (token, head)); pg_lightning_attention runs the recurrence over them. */
long long pg_lightning_record_floats(int n_tokens, int heads, int dim, int vdim);
int pg_lightning_prep(float* rec, const void* proj, int ld, int q_col0, int k_col0, int v_col0, int n_tokens, int heads,
                      int dim, int vdim, int dtype, void* stream);
int pg_lightning_attention(float* out, float* state, const float* rec, const float* decay, const int32_t* segs, int n_segs,
                           int heads, int dim, int vdim, void* stream);

/* ---- latent attention ------------------------------------------------------------------------------------------
 * pg_latent_prep: from the fused projection row [.. dq (q_rank) .. dkv (kv_rank + rot_dim) ..]:
 *   cq_out[t] = RMS(dq) * w_q (model dtype, packed [n_tokens, q_rank]);
 *   pool row of (tok_slot, tok_pos) = [RMS(dkv[:kv_rank]) * w_kv | rotary(dkv[kv_rank:]) | zeros up to ld_pool]
 *   (pairs (2i, 2i+1), angle pos * freq[i], cos and sin times mag, fp32).
 * pg_rotary_cols: the same rotation of rot_dim columns of every head of a row into another matrix.
 * pg_head_gemm: out[t, h*out_head_stride + n] = sum_k A[t, h*a_head_stride + k] W[h][n][k] for all heads (W is
 *   [heads][N][K]), times sigmoid(gate[t, h*N + n]) when a gate is given; fp32 accumulation, one rounding.
 * pg_attention_ragged_sink: pg_attention_ragged_ex with explicit row strides of the two pools (0: packed) and
 *   sink (device fp32 [n_heads], may be NULL): exp(sink[h]) is added once to the softmax denominator.
 * pg_concat_cast: out[r] = [a[r] | b[r]] of two fp32 [rows, D] matrices in the model dtype. */
int pg_latent_prep(void* cq_out, const void* proj, int ld, int dq_col0, int q_rank, const void* w_q, int dkv_col0,
                   int kv_rank, const void* w_kv, int rot_dim, const float* freq, float mag, float eps, void* pool,
                   int ld_pool, const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                   const int32_t* tok_pos, int n_tokens, int dtype, void* stream);
int pg_rotary_cols(void* dst, int ld_dst, int dst_col0, int dst_head_stride, const void* src, int ld_src, int src_col0,
                   int src_head_stride, int heads, int rot_dim, const float* freq, float mag, const int32_t* tok_pos,
                   int n_tokens, int dtype, void* stream);
int pg_head_gemm(void* out, int ldo, int out_head_stride, const void* A, int lda, int a_head_stride, const void* W,
                 const void* gate, int ld_gate, int n_rows, int heads, int N, int K, int dtype, void* stream);
/* pg_head_gemm_ex: impl 0 = the grouped tcgen05 kernel in its per-head mode for 16-bit row counts from 64 on (every
 * stride and size a multiple of 8; its waits are bounded, *err_flag becomes 2 if one gives up), else the fp32-FMA
 * kernels; 1 = the fp32-FMA kernels (pg_head_gemm); 2 = the tensor-core kernel or an error. */
int pg_head_gemm_ex(void* out, int ldo, int out_head_stride, const void* A, int lda, int a_head_stride, const void* W,
                    const void* gate, int ld_gate, int n_rows, int heads, int N, int K, int impl, int* err_flag, int dtype,
                    void* stream);
int pg_attention_ragged_sink(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                             int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                             const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                             const int32_t* tok_pos, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                             float scale, int window, int keep_first, const float* slopes, int sigmoid_weights,
                             const float* head_bias, const float* sink, float out_scale, float* ws, long long ws_floats,
                             int dtype, void* stream);
int pg_concat_cast(void* out, const float* a, const float* b, int rows, int D, int dtype, void* stream);
/* pg_attention_ragged_tc_ex with explicit row strides of the two pools (0: packed; multiples of 8 elements) and the
 * softmax sink of pg_attention_ragged_sink. */
int pg_attention_ragged_tc_sink(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                long long pool_rows, const int32_t* page_table, int pt_stride, int page_size,
                                const int32_t* tiles, int n_tiles, int n_tokens, int n_heads, int n_kv_heads, int dim,
                                int vdim, float scale, int window, int keep_first, const float* slopes,
                                int sigmoid_weights, const float* head_bias, const float* sink, float out_scale,
                                int* err_flag, int dtype, void* stream);

/* ---- norms stored around zero, short convolutions over time, per-head norms with rotated values, blocked masks,
 * ---- the selective state-space mixer ------------------------------------------------------------------------------
 * pg_group_rmsnorm_ex: pg_group_rmsnorm with two switches.  one_plus != 0: the weight is stored around zero and the
 *   row is multiplied by 1 + w (the sum in fp32).  out_f32 != 0: out is fp32 [rows, D], not rounded (for a consumer
 *   that goes on in fp32).
 * pg_time_conv_residual: out[t] = in[t] + sum_j w[:, j] in_(t - taps + 1 + j) per channel, a causal convolution over
 *   the positions of the token's sequence (w [C][taps], model dtype, last column = the current token; in fp32
 *   [n_tokens, C]; out model dtype).  Inputs of earlier positions are the rows right before the token while they
 *   belong to the same sequence (same tok_slot), beyond that the sequence's state [slots][taps - 1][C] fp32 (entry
 *   taps - 2 the most recent; zeros for a new sequence).
 * pg_time_conv_state: after the step's readers: for every segment {slot, first row, tokens} the state becomes the last
 *   taps - 1 inputs of [old state ; rows of the segment], the rows read from src (fp32 when src_f32 != 0, else the
 *   model dtype) at columns col0 .. col0 + C of rows with stride ld.  Segments of 0 tokens are skipped.
 * pg_headnorm_rotary_append: per token, from one fused projection row: every query / key head is divided by its root
 *   mean square over dim and multiplied by q_w / k_w (dim entries shared by the heads; NULL: no norm), then rotated as
 *   in pg_rotary_append (no magnitude); every value head is divided by its root mean square over vdim when v_norm != 0
 *   and, with v_freq (device float [vdim / 2]), rotated over all its columns by position * v_freq[m] (pairs (2m, 2m+1)
 *   when v_interleaved != 0, else (m, m + vdim / 2)).  Queries to q_out (packed), keys and values to the paged pools.
 * pg_attention_ragged_masked: pg_attention_ragged_sink with chunk > 0: key j is visible to the query at position i only
 *   if j <= i and floor(i / chunk) == floor(j / chunk) (together with the window when one is given), and out_rot
 *   (device float [vdim / 2], may be NULL): every head's result is turned back by -i * out_rot[m] in the pair layout
 *   out_rot_interleaved names, in fp32 before the gate and the single rounding (values cached rotated by their
 *   positions).
 * pg_relu2: out = max(z, 0)^2 (out may alias z).
 * pg_ssm_prep / pg_gate_groupnorm: the state-space mixer around the decayed linear-attention scan.  From the fused
 *   projection row [z | x | B | C | dt] (x, B, C from column xbc_col0, dt from dt_col0): causal convolution (conv_w
 *   [channels][taps], conv_b, channels = heads * vdim + 2 * groups * state; state of earlier inputs as for
 *   pg_time_conv_residual, kept by pg_time_conv_state over the projection's columns) and silu on x, B, C;
 *   step = softplus(dt + dt_bias[h]); one fp32 record per (token, head): [C | step * B | x | exp(-exp(a_log[h]) step),
 *   0, 0, 0] with C, B padded to state rounded up to 4 floats and x to vdim likewise: the records of
 *   pg_lightning_attention_ex with a decay per token.  rec holds pg_ssm_record_floats() floats.
 *   pg_gate_groupnorm: out = RMS over each of `groups` equal parts of (y * silu(z)) times w (w may be NULL); y fp32
 *   [n_tokens, cols] packed, z model dtype with row stride ld_z.
 * pg_lightning_attention_ex: pg_lightning_attention with skip (device float [heads], may be NULL: skip[h] * v is added
 *   to the output) and, when decay == NULL, records that carry [decay, 0, 0, 0] after the values: S <- decay_t S + k v^T. */
int pg_group_rmsnorm_ex(void* out, float* x, const void* add_a, int lda, const void* add_b, int ldb, const void* w,
                        const int32_t* rows_idx, int rows, int D, int groups, float eps, int one_plus, int out_f32,
                        int dtype, void* stream);
int pg_time_conv_residual(void* out, const float* in, const void* w, const float* state, const int32_t* tok_slot,
                          int n_tokens, int C, int taps, int dtype, void* stream);
/* pg_norm_time_conv: pg_group_rmsnorm_ex (one group, fp32) + pg_time_conv_residual + pg_time_conv_state in one pass and a
 * small second launch: x_out = x_in + y (y may be NULL; x_out must not alias x_in), out = n + conv(n) with
 * n = RMS(x_out) * (w_norm or 1 + w_norm), then the sequences' states [slots][taps - 1][D] of normed rows are brought up
 * to the end of the step's segments.  taps <= 8. */
int pg_norm_time_conv(void* out, float* x_out, const float* x_in, const void* y, int ldy, const void* w_norm, int one_plus,
                      float eps, const void* w_conv, float* state, const int32_t* tok_slot, const int32_t* segs, int n_segs,
                      int n_tokens, int D, int taps, int dtype, void* stream);
int pg_time_conv_state(float* state, const void* src, int ld, int col0, int src_f32, const int32_t* segs, int n_segs,
                       int C, int taps, int dtype, void* stream);
int pg_headnorm_rotary_append(void* q_out, const void* proj, int ld, int q_col0, int n_heads, int k_col0, int n_kv_heads,
                              int dim, int v_col0, int vdim, const void* q_w, const void* k_w, float eps,
                              const float* freq, int rot_dims, int interleaved, int v_norm, const float* v_freq,
                              int v_interleaved, void* k_pool, void* v_pool, const int32_t* page_table, int pt_stride,
                              int page_size, const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int dtype,
                              void* stream);
int pg_attention_ragged_masked(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                               int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                               const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                               const int32_t* tok_pos, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
                               float scale, int window, int keep_first, int chunk, const float* slopes,
                               int sigmoid_weights, const float* head_bias, const float* sink, const float* out_rot,
                               int out_rot_interleaved, float out_scale, float* ws, long long ws_floats, int dtype,
                               void* stream);
/* pg_attention_ragged_tc_sink with the block mask and the turning back of pg_attention_ragged_masked (vdim is a multiple
 * of 64 here, so both pair layouts fall on whole 32-column loads of the accumulator). */
int pg_attention_ragged_tc_masked(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                  int gate_per_head, const void* k_pool, int ld_k, const void* v_pool, int ld_v,
                                  long long pool_rows, const int32_t* page_table, int pt_stride, int page_size,
                                  const int32_t* tiles, int n_tiles, int n_tokens, int n_heads, int n_kv_heads, int dim,
                                  int vdim, float scale, int window, int keep_first, int chunk, const float* slopes,
                                  int sigmoid_weights, const float* head_bias, const float* sink, const float* out_rot,
                                  int out_rot_interleaved, float out_scale, int* err_flag, int dtype, void* stream);
int pg_relu2(void* out, const void* z, long long n, int dtype, void* stream);
long long pg_ssm_record_floats(int n_tokens, int heads, int vdim, int state);
int pg_ssm_prep(float* rec, const void* proj, int ld, int xbc_col0, int dt_col0, const void* conv_w, const void* conv_b,
                const float* conv_state, const float* dt_bias, const float* a_log, const int32_t* tok_slot, int n_tokens,
                int heads, int vdim, int state, int groups, int taps, int dtype, void* stream);
int pg_gate_groupnorm(void* out, int ld_out, const float* y, const void* z, int ld_z, const void* w, int n_tokens, int cols,
                      int groups, float eps, int dtype, void* stream);
int pg_lightning_attention_ex(float* out, float* state, const float* rec, const float* decay, const float* skip,
                              const int32_t* segs, int n_segs, int heads, int dim, int vdim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PG_B200_H */
