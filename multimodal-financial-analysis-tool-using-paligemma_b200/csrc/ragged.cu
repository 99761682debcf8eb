// Row kernels for ragged token batches (decoder-only models served through the slot scheduler): every token t of a
// step carries the page-table row of its sequence (tok_slot[t]) and its position in that sequence (tok_pos[t]), so
// portions of prompts and single decoded tokens of different sequences run side by side in one launch.
//
// The residual stream of these models is fp32 whatever the model dtype: sums into it, norms and their statistics
// are evaluated in fp32 and only the normalised rows (the GEMM operands) are rounded to the model dtype.
#include "common.cuh"

namespace pg {

// ------------------------------------------------------------------ token embedding + learned position vector
template <typename T>
__global__ void embed_pos_kernel(float* __restrict__ x, const int64_t* __restrict__ ids, const int32_t* __restrict__ pos,
                                 const T* __restrict__ emb, const T* __restrict__ pos_emb, int D, int64_t vocab,
                                 int max_pos, float emb_scale, int* err_flag) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int64_t id = ids[t];
  const int p = pos ? pos[t] : 0;
  const bool ok = id >= 0 && id < vocab && (!pos_emb || (p >= 0 && p < max_pos));
  if (!ok && err_flag && threadIdx.x == 0) *err_flag = 1;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float v = 0.f;
    if (ok) {
      v = to_f<T>(emb[(size_t)id * D + c]) * emb_scale;
      if (pos_emb) v += to_f<T>(pos_emb[(size_t)p * D + c]);
    }
    x[(size_t)t * D + c] = v;
  }
}

// ------------------------------------------------------------------ residual sum + RMS norm in groups
// One warp per (row, group).  x[row] += a[row] + b[row] first (either may be absent; the sum is written back), then
// each of the `groups` equal consecutive parts of the row is divided by its own sqrt(mean(part^2) + eps) and the
// whole is multiplied by w (by 1 + w when the weight is stored around zero: one_plus).  rows_idx (optional) picks the
// input rows; output rows are packed, in the model dtype or (TO = float) unrounded for a consumer that goes on in fp32.
template <typename T, typename TO>
__global__ void group_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ x, const T* __restrict__ a, int lda,
                                     const T* __restrict__ b, int ldb, const T* __restrict__ w,
                                     const int32_t* __restrict__ rows_idx, int rows, int D, int groups, float eps,
                                     int one_plus) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= rows * groups) return;
  const int r = item / groups, g = item % groups;
  const int src = rows_idx ? rows_idx[r] : r;
  const int gs = D / groups;
  float* xr = x + (size_t)src * D + g * gs;
  float ss = 0.f;
  for (int c = lane; c < gs; c += 32) {
    float v = xr[c];
    if (a || b) {
      float add = 0.f;
      if (a) add += to_f<T>(a[(size_t)src * lda + g * gs + c]);
      if (b) add += to_f<T>(b[(size_t)src * ldb + g * gs + c]);
      v += add;
      xr[c] = v;
    }
    ss += v * v;
  }
  if (!out) return;
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)gs + eps);
  TO* o = out + (size_t)r * D + g * gs;
  const float w0 = one_plus ? 1.f : 0.f;
  for (int c = lane; c < gs; c += 32) o[c] = from_f<TO>(xr[c] * inv * (w0 + to_f<T>(w[g * gs + c])));
}

// ------------------------------------------------------------------ query / key norm over the whole projection + cache append
// One CTA per token.  proj row = [.. q (q_cols) .. k (k_cols) .. v (v_cols) ..] at the given column offsets.
// q_out = q / rms(q) * q_w over ALL q columns at once (not per head); the key row likewise, written with the value
// row into the paged pools at (tok_slot, tok_pos).  k_cols == 0: a layer that reads another layer's keys and values.
template <typename T>
__global__ void qknorm_append_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int ld, int q_col0, int q_cols,
                                     int k_col0, int k_cols, int v_col0, int v_cols, const T* __restrict__ q_w,
                                     const T* __restrict__ k_w, float eps, T* __restrict__ k_pool,
                                     T* __restrict__ v_pool, const int32_t* __restrict__ page_table, int pt_stride,
                                     int page_size, const int32_t* __restrict__ tok_slot,
                                     const int32_t* __restrict__ tok_pos) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  float ss = 0.f;
  for (int c = threadIdx.x; c < q_cols; c += blockDim.x) { const float v = to_f<T>(row[q_col0 + c]); ss += v * v; }
  ss = block_sum(ss, red);
  float inv = q_w ? 1.f / sqrtf(ss / (float)q_cols + eps) : 1.f;
  for (int c = threadIdx.x; c < q_cols; c += blockDim.x)
    q_out[(size_t)t * q_cols + c] = from_f<T>(to_f<T>(row[q_col0 + c]) * inv * (q_w ? to_f<T>(q_w[c]) : 1.f));
  if (k_cols == 0) return;
  const int p = tok_pos[t];
  const size_t slot_row = (size_t)page_table[(size_t)tok_slot[t] * pt_stride + p / page_size] * page_size + p % page_size;
  ss = 0.f;
  for (int c = threadIdx.x; c < k_cols; c += blockDim.x) { const float v = to_f<T>(row[k_col0 + c]); ss += v * v; }
  ss = block_sum(ss, red);
  inv = k_w ? 1.f / sqrtf(ss / (float)k_cols + eps) : 1.f;
  for (int c = threadIdx.x; c < k_cols; c += blockDim.x)
    k_pool[slot_row * k_cols + c] = from_f<T>(to_f<T>(row[k_col0 + c]) * inv * (k_w ? to_f<T>(k_w[c]) : 1.f));
  for (int c = threadIdx.x; c < v_cols; c += blockDim.x) v_pool[slot_row * v_cols + c] = row[v_col0 + c];
}

// ------------------------------------------------------------------ xIELU activation
// z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2.  (p, q) = pq[0..1].
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void xielu_kernel(T* __restrict__ out, const T* __restrict__ z, const T* __restrict__ pq, long long n, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec<T>::N;
  const float ap = softplus_f(to_f<T>(pq[0])), an = 0.5f + softplus_f(to_f<T>(pq[1]));
  auto act = [&](float v) { return v > 0.f ? ap * v * v + 0.5f * v : an * (expm1f(v) - v) + 0.5f * v; };
  const long long stride = (long long)gridDim.x * blockDim.x, first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (vec) {   // 16-byte accesses (n a multiple of the vector width, aligned pointers: checked on the host)
    for (long long i = first; i < n / V; i += stride) {
      float f[V];
      unpack<T>(*reinterpret_cast<const uint4*>(z + i * V), f);
#pragma unroll
      for (int k = 0; k < V; ++k) f[k] = act(f[k]);
      *reinterpret_cast<uint4*>(out + i * V) = pack<T>(f);
    }
    return;
  }
  for (long long i = first; i < n; i += stride) out[i] = from_f<T>(act(to_f<T>(z[i])));
}

// ------------------------------------------------------------------ gated pairing of a stacked [gate | up] row
// GELU == false: silu(gate) * up; GELU == true: gelu_tanh(gate) * up.  The activation is rounded to the model dtype
// before the product, as the GEMM epilogues do.
template <typename T, bool GELU>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int rows, int F) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)rows * F;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F, c = i % F;
    const float g = to_f<T>(gu[r * 2 * F + c]), u = to_f<T>(gu[r * 2 * F + F + c]);
    out[i] = from_f<T>(rnd<T>(GELU ? gelu_tanh(g) : g / (1.f + expf(-g))) * u);
  }
}

// The clamped pairing of a stacked [gate | up] row: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g sigmoid(alpha g) (u + 1); the activation is rounded to the model dtype before the product.
template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ gu, int rows, int F, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)rows * F;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F, c = i % F;
    const float g = fminf(to_f<T>(gu[r * 2 * F + c]), limit);
    const float u = fminf(fmaxf(to_f<T>(gu[r * 2 * F + F + c]), -limit), limit);
    out[i] = from_f<T>(rnd<T>(g / (1.f + expf(-alpha * g))) * (u + 1.f));
  }
}

// ------------------------------------------------------------------ bias + rotary positions + value mixing + cache append
// One CTA per token.  proj row = [.. q (H heads x dim) .. k (G x dim) .. v (G x vdim) ..] at the given column offsets.
// Optional biases (model dtype) are added in fp32 first.  The first rot_dims columns of every query and key head are
// rotated as pairs: interleaved != 0 pairs column 2i with 2i + 1, otherwise column i with i + rot_dims / 2; the pair
// (a, b) at position p becomes mag * (a cos t - b sin t, b cos t + a sin t) with t = p * freq[i], evaluated in fp32
// with the full-range sincosf; the other columns pass unchanged.  v_first != NULL: the value row becomes
// (1 - lambda) v + lambda v_first[t] (the values of the same token from an earlier layer) before it is cached.
// Query rows go to q_out (packed), key and value rows to the paged pools at (tok_slot, tok_pos).
template <typename T>
__global__ void rotary_append_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int ld, int q_col0, int H,
                                     int k_col0, int G, int dim, int v_col0, int vdim, const T* __restrict__ q_bias,
                                     const T* __restrict__ k_bias, const T* __restrict__ v_bias,
                                     const float* __restrict__ freq, int rot_dims, float mag, int interleaved,
                                     const T* __restrict__ v_first, int ld_vf, float lambda, T* __restrict__ k_pool,
                                     T* __restrict__ v_pool, const int32_t* __restrict__ page_table, int pt_stride,
                                     int page_size, const int32_t* __restrict__ tok_slot,
                                     const int32_t* __restrict__ tok_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  const int p = tok_pos[t];
  const float fp = (float)p;
  const size_t slot_row = (size_t)page_table[(size_t)tok_slot[t] * pt_stride + p / page_size] * page_size + p % page_size;
  T* kdst = k_pool + slot_row * ((size_t)G * dim);
  T* qdst = q_out + (size_t)t * H * dim;
  const int half = rot_dims >> 1, rest = dim - rot_dims;
  // rotated pairs of the query heads, then of the key heads
  for (int idx = threadIdx.x; idx < (H + G) * half; idx += blockDim.x) {
    const bool is_k = idx >= H * half;
    const int li = is_k ? idx - H * half : idx, head = li / half, i = li % half;
    const int c0 = interleaved ? 2 * i : i, c1 = interleaved ? 2 * i + 1 : i + half;
    const int base = head * dim;
    const T* src = row + (is_k ? k_col0 : q_col0) + base;
    const T* bias = is_k ? k_bias : q_bias;
    float a = to_f<T>(src[c0]), b = to_f<T>(src[c1]);
    if (bias) { a += to_f<T>(bias[base + c0]); b += to_f<T>(bias[base + c1]); }
    float sn, cs;
    sincosf(fp * freq[i], &sn, &cs);
    sn *= mag; cs *= mag;
    T* dst = (is_k ? kdst : qdst) + base;
    dst[c0] = from_f<T>(a * cs - b * sn);
    dst[c1] = from_f<T>(b * cs + a * sn);
  }
  // columns that are not rotated
  for (int idx = threadIdx.x; idx < (H + G) * rest; idx += blockDim.x) {
    const bool is_k = idx >= H * rest;
    const int li = is_k ? idx - H * rest : idx, c = (li / rest) * dim + rot_dims + li % rest;
    const T* bias = is_k ? k_bias : q_bias;
    float a = to_f<T>(row[(is_k ? k_col0 : q_col0) + c]);
    if (bias) a += to_f<T>(bias[c]);
    (is_k ? kdst : qdst)[c] = from_f<T>(a);
  }
  T* vdst = v_pool + slot_row * ((size_t)G * vdim);
  const T* vf = v_first ? v_first + (size_t)t * ld_vf : nullptr;
  for (int c = threadIdx.x; c < G * vdim; c += blockDim.x) {
    float v = to_f<T>(row[v_col0 + c]);
    if (v_bias) v += to_f<T>(v_bias[c]);
    if (vf) v = (1.f - lambda) * v + lambda * to_f<T>(vf[c]);
    vdst[c] = from_f<T>(v);
  }
}

// ------------------------------------------------------------------ output norm + layer scale + residual sum + next input norm
// One warp per row.  x[r] += scale (.) (y[r] / sqrt(mean(y[r]^2) + eps) * w_post) with y a sublayer's output (model
// dtype), w_post its output-norm weight and `scale` a per-channel layer scale (NULL: none); then, when out != NULL,
// out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w_next: the next sublayer's input.  Statistics and sums in fp32.
template <typename T>
__global__ void postnorm_residual_kernel(T* __restrict__ out, float* __restrict__ x, const T* __restrict__ y, int ldy,
                                         const T* __restrict__ w_post, const T* __restrict__ scale,
                                         const T* __restrict__ w_next, int rows, int D, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* yr = y + (size_t)r * ldy;
  float* xr = x + (size_t)r * D;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) { const float v = to_f<T>(yr[c]); ss += v * v; }
  ss = warp_sum(ss);
  const float inv_y = 1.f / sqrtf(ss / (float)D + eps);
  float sx = 0.f;
  for (int c = lane; c < D; c += 32) {
    float v = to_f<T>(yr[c]) * inv_y * to_f<T>(w_post[c]);
    if (scale) v *= to_f<T>(scale[c]);
    v += xr[c];
    xr[c] = v;
    sx += v * v;
  }
  if (!out) return;
  sx = warp_sum(sx);
  const float inv_x = 1.f / sqrtf(sx / (float)D + eps);
  T* o = out + (size_t)r * D;
  for (int c = lane; c < D; c += 32) o[c] = from_f<T>(xr[c] * inv_x * to_f<T>(w_next[c]));
}

// The same for a handful of rows (decode-sized steps): one CTA per row, a thread keeps its PER elements of the row
// in registers between the statistics and the writes (D <= PER * blockDim.x).
template <typename T, int PER>
__global__ void __launch_bounds__(256)
postnorm_residual_row_kernel(T* __restrict__ out, float* __restrict__ x, const T* __restrict__ y, int ldy,
                             const T* __restrict__ w_post, const T* __restrict__ scale, const T* __restrict__ w_next,
                             int D, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  float wp[PER], sc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {                  // weights do not depend on the preceding kernel
    const int c = threadIdx.x + i * blockDim.x;
    wp[i] = c < D ? to_f<T>(w_post[c]) : 0.f;
    sc[i] = (c < D && scale) ? to_f<T>(scale[c]) : 1.f;
  }
  pdl_wait();
  const int r = blockIdx.x;
  const T* yr = y + (size_t)r * ldy;
  float* xr = x + (size_t)r * D;
  float yv[PER], xv[PER], ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    yv[i] = c < D ? to_f<T>(yr[c]) : 0.f;
    xv[i] = c < D ? xr[c] : 0.f;
    ss += yv[i] * yv[i];
  }
  ss = block_sum(ss, red);
  const float inv_y = 1.f / sqrtf(ss / (float)D + eps);
  float sx = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    xv[i] += yv[i] * inv_y * wp[i] * sc[i];
    if (c < D) { xr[c] = xv[i]; sx += xv[i] * xv[i]; }
  }
  if (!out) return;
  sx = block_sum(sx, red);
  const float inv_x = 1.f / sqrtf(sx / (float)D + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < D) out[(size_t)r * D + c] = from_f<T>(xv[i] * inv_x * to_f<T>(w_next[c]));
  }
}

// ------------------------------------------------------------------ per-head norms + rotary positions (keys, queries AND values) + cache append
// One CTA per token, one warp per head (query heads, then key heads, then value heads).  Every query / key head is
// divided by its own root mean square over `dim` and multiplied by a weight of `dim` entries shared by the heads
// (q_w / k_w NULL: no norm), then its first rot_dims columns are rotated by position * freq[i] (pairs (2i, 2i+1) when
// interleaved, else (i, i + rot_dims / 2)).  Every value head is divided by its root mean square over vdim when v_norm
// is set (no weight) and, with v_freq, rotated over ALL its columns by position * v_freq[m] in the layout v_interleaved
// names; the attention that reads such values turns its result back by the query's position.  Norm statistics, angles
// and the rotation are fp32; one rounding when the row is stored.
template <typename T>
__global__ void headnorm_rotary_append_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int ld, int q_col0, int H,
                                              int k_col0, int G, int dim, int v_col0, int vdim, const T* __restrict__ q_w,
                                              const T* __restrict__ k_w, float eps, const float* __restrict__ freq,
                                              int rot_dims, int interleaved, int v_norm, const float* __restrict__ v_freq,
                                              int v_interleaved, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                              const int32_t* __restrict__ page_table, int pt_stride, int page_size,
                                              const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* row = proj + (size_t)t * ld;
  const int p = tok_pos[t];
  const float fp = (float)p;
  const size_t slot_row = (size_t)page_table[(size_t)tok_slot[t] * pt_stride + p / page_size] * page_size + p % page_size;
  for (int item = warp; item < H + 2 * G; item += warps) {
    const int kind = item < H ? 0 : (item < H + G ? 1 : 2);
    const int head = kind == 0 ? item : (kind == 1 ? item - H : item - H - G);
    const int n = kind == 2 ? vdim : dim;
    const T* src = row + (kind == 0 ? q_col0 : (kind == 1 ? k_col0 : v_col0)) + head * n;
    T* dst = kind == 0 ? q_out + (size_t)t * H * dim + head * dim
                       : (kind == 1 ? k_pool + slot_row * ((size_t)G * dim) + head * dim
                                    : v_pool + slot_row * ((size_t)G * vdim) + head * vdim);
    const T* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
    const bool normed = kind == 2 ? v_norm != 0 : w != nullptr;
    const float* f = kind == 2 ? v_freq : freq;
    const int rd = kind == 2 ? (v_freq ? vdim & ~1 : 0) : rot_dims, il = kind == 2 ? v_interleaved : interleaved;
    float inv = 1.f;
    if (normed) {
      float ss = 0.f;
      for (int c = lane; c < n; c += 32) { const float v = to_f<T>(src[c]); ss += v * v; }
      inv = 1.f / sqrtf(warp_sum(ss) / (float)n + eps);
    }
    const int half = rd >> 1;
    for (int i = lane; i < half; i += 32) {
      const int c0 = il ? 2 * i : i, c1 = il ? 2 * i + 1 : i + half;
      const float a = to_f<T>(src[c0]) * inv * (w ? to_f<T>(w[c0]) : 1.f), b = to_f<T>(src[c1]) * inv * (w ? to_f<T>(w[c1]) : 1.f);
      float sn, cs;
      sincosf(fp * f[i], &sn, &cs);
      dst[c0] = from_f<T>(a * cs - b * sn);
      dst[c1] = from_f<T>(b * cs + a * sn);
    }
    for (int c = rd + lane; c < n; c += 32) dst[c] = from_f<T>(to_f<T>(src[c]) * inv * (w ? to_f<T>(w[c]) : 1.f));
  }
}

// ------------------------------------------------------------------ squared ReLU
template <typename T>
__global__ void relu2_kernel(T* __restrict__ out, const T* __restrict__ z, long long n, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec<T>::N;
  const long long stride = (long long)gridDim.x * blockDim.x, first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (vec) {
    for (long long i = first; i < n / V; i += stride) {
      float f[V];
      unpack<T>(*reinterpret_cast<const uint4*>(z + i * V), f);
#pragma unroll
      for (int k = 0; k < V; ++k) { const float r = fmaxf(f[k], 0.f); f[k] = r * r; }
      *reinterpret_cast<uint4*>(out + i * V) = pack<T>(f);
    }
    return;
  }
  for (long long i = first; i < n; i += stride) { const float r = fmaxf(to_f<T>(z[i]), 0.f); out[i] = from_f<T>(r * r); }
}

}  // namespace pg

using namespace pg;

extern "C" int pg_embed_pos(float* x, const int64_t* ids, const int32_t* positions, const void* emb,
                            const void* pos_emb, int n_tokens, int D, int64_t vocab, int max_pos, float emb_scale,
                            int* err_flag, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("embed_pos", embed_pos_kernel<T>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, x, ids, positions,
                      (const T*)emb, (const T*)pos_emb, D, vocab, max_pos, emb_scale, err_flag);
  });
  return PG_OK;
}

extern "C" int pg_group_rmsnorm(void* out, float* x, const void* add_a, int lda, const void* add_b, int ldb,
                                const void* w, const int32_t* rows_idx, int rows, int D, int groups, float eps,
                                int dtype, void* stream) {
  return pg_group_rmsnorm_ex(out, x, add_a, lda, add_b, ldb, w, rows_idx, rows, D, groups, eps, 0, 0, dtype, stream);
}

extern "C" int pg_group_rmsnorm_ex(void* out, float* x, const void* add_a, int lda, const void* add_b, int ldb,
                                   const void* w, const int32_t* rows_idx, int rows, int D, int groups, float eps,
                                   int one_plus, int out_f32, int dtype, void* stream) {
  if (rows <= 0) return PG_OK;
  PG_REQUIRE(groups >= 1 && D % groups == 0, "group_rmsnorm: D=%d is not a multiple of groups=%d", D, groups);
  PG_REQUIRE(!out || w, "group_rmsnorm: a normalised output needs a weight");
  PG_REQUIRE(!rows_idx || (!add_a && !add_b), "group_rmsnorm: the residual sum takes all rows (no row index)");
  const int warps = 8;
  PG_DISPATCH_DTYPE(dtype, T, {
    if (out_f32)
      return launch_pdl("group_rmsnorm", group_rmsnorm_kernel<T, float>, dim3(cdiv((long long)rows * groups, warps)),
                        dim3(warps * 32), 0, (cudaStream_t)stream, (float*)out, x, (const T*)add_a, lda, (const T*)add_b, ldb,
                        (const T*)w, rows_idx, rows, D, groups, eps, one_plus);
    return launch_pdl("group_rmsnorm", group_rmsnorm_kernel<T, T>, dim3(cdiv((long long)rows * groups, warps)), dim3(warps * 32),
                      0, (cudaStream_t)stream, (T*)out, x, (const T*)add_a, lda, (const T*)add_b, ldb, (const T*)w, rows_idx,
                      rows, D, groups, eps, one_plus);
  });
  return PG_OK;
}

extern "C" int pg_qknorm_append(void* q_out, const void* proj, int ld, int q_col0, int q_cols, int k_col0, int k_cols,
                                int v_col0, int v_cols, const void* q_w, const void* k_w, float eps, void* k_pool,
                                void* v_pool, const int32_t* page_table, int pt_stride, int page_size,
                                const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(k_cols == 0 || (k_pool && v_pool && page_table && tok_slot && tok_pos && page_size > 0),
             "qknorm_append: a layer with keys of its own needs the pools and the token map");
  PG_DISPATCH_DTYPE(dtype, T, {
    // a handful of tokens (decode steps): wide CTAs, so that a row is a few loads per thread
    const int threads = n_tokens <= 64 ? (q_cols >= 2048 ? 512 : 256) : 128;
    return launch_pdl("qknorm_append", qknorm_append_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream,
                      (T*)q_out, (const T*)proj, ld, q_col0, q_cols, k_col0, k_cols, v_col0, v_cols, (const T*)q_w,
                      (const T*)k_w, eps, (T*)k_pool, (T*)v_pool, page_table, pt_stride, page_size, tok_slot, tok_pos);
  });
  return PG_OK;
}

extern "C" int pg_xielu(void* out, const void* z, const void* pq, long long n, int dtype, void* stream) {
  if (n <= 0) return PG_OK;
  PG_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = Vec<T>::N;
    const int vec = (n % V == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)z % 16) == 0) ? 1 : 0;
    const long long work = vec ? n / V : n;
    const int blocks = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    return launch_pdl("xielu", xielu_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)z,
                      (const T*)pq, n, vec);
  });
  return PG_OK;
}

extern "C" int pg_swiglu(void* out, const void* gate_up, int rows, int F, int dtype, void* stream) {
  if (rows <= 0 || F <= 0) return PG_OK;
  const long long n = (long long)rows * F;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("swiglu", swiglu_kernel<T, false>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                      (const T*)gate_up, rows, F);
  });
  return PG_OK;
}

extern "C" int pg_glu_clamped(void* out, const void* gate_up, int rows, int F, float limit, float alpha, int dtype,
                              void* stream) {
  if (rows <= 0 || F <= 0) return PG_OK;
  const long long n = (long long)rows * F;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("glu_clamped", glu_clamped_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                      (const T*)gate_up, rows, F, limit, alpha);
  });
  return PG_OK;
}

extern "C" int pg_geglu(void* out, const void* gate_up, int rows, int F, int dtype, void* stream) {
  if (rows <= 0 || F <= 0) return PG_OK;
  const long long n = (long long)rows * F;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("geglu", swiglu_kernel<T, true>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                      (const T*)gate_up, rows, F);
  });
  return PG_OK;
}

extern "C" int pg_rotary_append(void* q_out, const void* proj, int ld, int q_col0, int n_heads, int k_col0,
                                int n_kv_heads, int dim, int v_col0, int vdim, const void* q_bias, const void* k_bias,
                                const void* v_bias, const float* freq, int rot_dims, float mag, int interleaved,
                                const void* v_first, int ld_vf, float lambda, void* k_pool, void* v_pool,
                                const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                                const int32_t* tok_pos, int n_tokens, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(k_pool && v_pool && page_table && tok_slot && tok_pos && page_size > 0, "rotary_append: pools and token map");
  PG_REQUIRE(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq),
             "rotary_append: %d rotated columns of %d (even, with a frequency table)", rot_dims, dim);
  PG_DISPATCH_DTYPE(dtype, T, {
    const int work = (n_heads + n_kv_heads) * dim;
    const int threads = work >= 4096 ? 512 : (work >= 1024 ? 256 : 128);
    return launch_pdl("rotary_append", rotary_append_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream,
                      (T*)q_out, (const T*)proj, ld, q_col0, n_heads, k_col0, n_kv_heads, dim, v_col0, vdim,
                      (const T*)q_bias, (const T*)k_bias, (const T*)v_bias, freq, rot_dims, mag, interleaved,
                      (const T*)v_first, ld_vf, lambda, (T*)k_pool, (T*)v_pool, page_table, pt_stride, page_size,
                      tok_slot, tok_pos);
  });
  return PG_OK;
}

extern "C" int pg_postnorm_residual(void* out, float* x, const void* y, int ldy, const void* w_post,
                                    const void* scale, const void* w_next, int rows, int D, float eps, int dtype,
                                    void* stream) {
  if (rows <= 0) return PG_OK;
  PG_REQUIRE(x && y && w_post && ldy >= D, "postnorm_residual: x, y and the output-norm weight are needed");
  PG_REQUIRE(!out || w_next, "postnorm_residual: a normalised output needs a weight");
  const int warps = 8;
  if (rows <= 64 && D <= 16 * 256) {               // decode-sized steps: a CTA per row, the row in registers
    const int per = D <= 1024 ? 4 : (D <= 2048 ? 8 : 16);
    PG_DISPATCH_DTYPE(dtype, T, {
      auto k = per == 4 ? postnorm_residual_row_kernel<T, 4> : (per == 8 ? postnorm_residual_row_kernel<T, 8> : postnorm_residual_row_kernel<T, 16>);
      return launch_pdl("postnorm_residual", k, dim3(rows), dim3(256), 0, (cudaStream_t)stream, (T*)out, x, (const T*)y, ldy,
                        (const T*)w_post, (const T*)scale, (const T*)w_next, D, eps);
    });
  }
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("postnorm_residual", postnorm_residual_kernel<T>, dim3(cdiv(rows, warps)), dim3(warps * 32), 0,
                      (cudaStream_t)stream, (T*)out, x, (const T*)y, ldy, (const T*)w_post, (const T*)scale,
                      (const T*)w_next, rows, D, eps);
  });
  return PG_OK;
}

extern "C" int pg_headnorm_rotary_append(void* q_out, const void* proj, int ld, int q_col0, int n_heads, int k_col0,
                                         int n_kv_heads, int dim, int v_col0, int vdim, const void* q_w, const void* k_w,
                                         float eps, const float* freq, int rot_dims, int interleaved, int v_norm,
                                         const float* v_freq, int v_interleaved, void* k_pool, void* v_pool,
                                         const int32_t* page_table, int pt_stride, int page_size, const int32_t* tok_slot,
                                         const int32_t* tok_pos, int n_tokens, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(q_out && proj && k_pool && v_pool && page_table && tok_slot && tok_pos && page_size > 0,
             "headnorm_rotary_append: pools and token map");
  PG_REQUIRE(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || freq),
             "headnorm_rotary_append: %d rotated columns of %d (even, with a frequency table)", rot_dims, dim);
  PG_REQUIRE(!v_freq || vdim % 2 == 0, "headnorm_rotary_append: rotated values need an even width, not %d", vdim);
  const int heads = n_heads + 2 * n_kv_heads;
  const int threads = heads >= 32 ? 1024 : (heads < 4 ? 128 : 32 * heads);     // a warp per head while a CTA can hold them
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("headnorm_rotary_append", headnorm_rotary_append_kernel<T>, dim3(n_tokens), dim3(threads), 0,
                      (cudaStream_t)stream, (T*)q_out, (const T*)proj, ld, q_col0, n_heads, k_col0, n_kv_heads, dim, v_col0,
                      vdim, (const T*)q_w, (const T*)k_w, eps, freq, rot_dims, interleaved, v_norm, v_freq, v_interleaved,
                      (T*)k_pool, (T*)v_pool, page_table, pt_stride, page_size, tok_slot, tok_pos);
  });
  return PG_OK;
}

extern "C" int pg_relu2(void* out, const void* z, long long n, int dtype, void* stream) {
  if (n <= 0) return PG_OK;
  PG_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = Vec<T>::N;
    const int vec = (n % V == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)z % 16) == 0) ? 1 : 0;
    const long long work = vec ? n / V : n;
    const int blocks = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    return launch_pdl("relu2", relu2_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)z, n, vec);
  });
  return PG_OK;
}
