// Latent attention for ragged token batches: queries and keys/values go through low-rank latents, and only the
// key/value latent c (RMS-normed) and one rotated key part shared by all heads are cached.  Attention then runs in the
// latent space ("absorbed" form): with the per-head key expansion K_h = W_uk,h c and value expansion V_h = W_uv,h c,
//     q_h . K_h(j) = (W_uk,h^T q_h) . c_j         and        sum_j p_j V_h(j) = W_uv,h (sum_j p_j c_j),
// so every head is a query of width kv_rank + rot_dim against ONE shared key row [c | k_rot] and one shared value row c:
// the ragged attention kernels serve it as grouped-query attention with a single key/value head whose value is a
// prefix of its key row.
//
//   latent_prep_kernel   (CTA per token)  c_q = RMS(dq) w_q  -> the query expansion's operand (model dtype);
//                                         c   = RMS(dkv[:kv_rank]) w_kv, k_rot = rotary(dkv[kv_rank:]) -> the paged
//                                         latent cache row [c | k_rot] of (sequence, position)
//   rotary_cols_kernel   (CTA per token)  the rotated part of every query head into the absorbed query rows
//   head_gemm_kernel     (64x64 tiles)    out[t, h] = A[t, h] W_h^T for every head h at once (fp32 accumulation), with an
//                                         optional sigmoid gate on the output: the absorption of W_uk into the queries
//                                         and the value expansion W_uv of the attended latents
//                                         (prompt-sized 16-bit steps: the grouped tcgen05 GEMM of the experts in its
//                                         per-head mode, moe_gemm_tcgen05.cu)
//   concat_cast_kernel                    [a | b] of two fp32 matrices as one model-dtype operand row
#include "common.cuh"

namespace pg {

// ------------------------------------------------------------------ query latent norm, key/value latent norm, rotated key, cache append
template <typename T>
__global__ void latent_prep_kernel(T* __restrict__ cq_out, const T* __restrict__ proj, int ld, int dq_col0, int q_rank,
                                   const T* __restrict__ w_q, int dkv_col0, int kv_rank, const T* __restrict__ w_kv,
                                   int rot_dim, const float* __restrict__ freq, float mag, float eps,
                                   T* __restrict__ pool, int ld_pool, const int32_t* __restrict__ page_table,
                                   int pt_stride, int page_size, const int32_t* __restrict__ tok_slot,
                                   const int32_t* __restrict__ tok_pos) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  const int p = tok_pos[t];
  const size_t slot_row = (size_t)page_table[(size_t)tok_slot[t] * pt_stride + p / page_size] * page_size + p % page_size;
  T* dst = pool + slot_row * (size_t)ld_pool;
  float ss = 0.f;
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) { const float v = to_f<T>(row[dq_col0 + c]); ss += v * v; }
  ss = block_sum(ss, red);
  const float inv_q = 1.f / sqrtf(ss / (float)q_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
    cq_out[(size_t)t * q_rank + c] = from_f<T>(to_f<T>(row[dq_col0 + c]) * inv_q * to_f<T>(w_q[c]));
  ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) { const float v = to_f<T>(row[dkv_col0 + c]); ss += v * v; }
  ss = block_sum(ss, red);
  const float inv_kv = 1.f / sqrtf(ss / (float)kv_rank + eps);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
    dst[c] = from_f<T>(to_f<T>(row[dkv_col0 + c]) * inv_kv * to_f<T>(w_kv[c]));
  const float fp = (float)p;
  for (int i = threadIdx.x; i < rot_dim / 2; i += blockDim.x) {
    const float a = to_f<T>(row[dkv_col0 + kv_rank + 2 * i]), b = to_f<T>(row[dkv_col0 + kv_rank + 2 * i + 1]);
    float sn, cs;
    sincosf(fp * freq[i], &sn, &cs);
    sn *= mag; cs *= mag;
    dst[kv_rank + 2 * i] = from_f<T>(a * cs - b * sn);
    dst[kv_rank + 2 * i + 1] = from_f<T>(b * cs + a * sn);
  }
  for (int c = kv_rank + rot_dim + threadIdx.x; c < ld_pool; c += blockDim.x) dst[c] = from_f<T>(0.f);
}

// ------------------------------------------------------------------ rotated columns of every head of a row
// dst[t, h * dst_hs + dst_col0 + (2i, 2i+1)] = rotation of src[t, h * src_hs + src_col0 + (2i, 2i+1)] by pos[t] * freq[i]
template <typename T>
__global__ void rotary_cols_kernel(T* __restrict__ dst, int ld_dst, int dst_col0, int dst_hs, const T* __restrict__ src,
                                   int ld_src, int src_col0, int src_hs, int heads, int rot_dim,
                                   const float* __restrict__ freq, float mag, const int32_t* __restrict__ tok_pos) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, half = rot_dim / 2;
  const float fp = (float)tok_pos[t];
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const T* s = src + (size_t)t * ld_src + h * src_hs + src_col0 + 2 * i;
    T* d = dst + (size_t)t * ld_dst + h * dst_hs + dst_col0 + 2 * i;
    const float a = to_f<T>(s[0]), b = to_f<T>(s[1]);
    float sn, cs;
    sincosf(fp * freq[i], &sn, &cs);
    sn *= mag; cs *= mag;
    d[0] = from_f<T>(a * cs - b * sn);
    d[1] = from_f<T>(b * cs + a * sn);
  }
}

// ------------------------------------------------------------------ one small GEMM per head, all heads in one launch
// out[t, h * o_hs + n] = sum_k A[t, h * a_hs + k] * W[(h * N + n) * K + k]   (* sigmoid(gate[t, h * N + n]))
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16, HG_THREADS = 256, HG_PAD = 4;

template <typename T>
__global__ void __launch_bounds__(HG_THREADS)
head_gemm_kernel(T* __restrict__ out, int ldo, int o_hs, const T* __restrict__ A, int lda, int a_hs,
                 const T* __restrict__ W, const T* __restrict__ gate, int ldg, int M, int N, int K) {
  __shared__ __align__(16) float As[HG_BK][HG_BM + HG_PAD];
  __shared__ __align__(16) float Bs[HG_BK][HG_BN + HG_PAD];
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.z, m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
  const T* Ah = A + (size_t)h * a_hs;
  const T* Wh = W + (size_t)h * N * K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HG_BK) {
    for (int idx = threadIdx.x; idx < HG_BM * HG_BK; idx += HG_THREADS) {
      const int r = idx / HG_BK, kk = idx % HG_BK;
      float a = 0.f, b = 0.f;
      if (k0 + kk < K) {
        if (m0 + r < M) a = to_f<T>(Ah[(size_t)(m0 + r) * lda + k0 + kk]);
        if (n0 + r < N) b = to_f<T>(Wh[(size_t)(n0 + r) * K + k0 + kk]);
      }
      As[kk][r] = a;
      Bs[kk][r] = b;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HG_BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (gate) v = rnd<T>(v) * (1.f / (1.f + expf(-to_f<T>(gate[(size_t)m * ldg + h * N + n]))));
      out[(size_t)m * ldo + h * o_hs + n] = from_f<T>(v);
    }
  }
}

// A handful of rows (decode-sized steps): the weights of a head are streamed once, a warp owns an output column n of
// a head and keeps one accumulator per row (up to HV_ROWS rows per launch slice).
constexpr int HV_ROWS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
head_gemv_kernel(T* __restrict__ out, int ldo, int o_hs, const T* __restrict__ A, int lda, int a_hs,
                 const T* __restrict__ W, const T* __restrict__ gate, int ldg, int M, int N, int K) {
  extern __shared__ float as[];                  // [rows][K] fp32 operand rows of this head
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.y, m0 = blockIdx.z * HV_ROWS, rows = min(HV_ROWS, M - m0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int idx = threadIdx.x; idx < rows * K; idx += blockDim.x) {
    const int r = idx / K, k = idx % K;
    as[idx] = to_f<T>(A[(size_t)(m0 + r) * lda + (size_t)h * a_hs + k]);
  }
  __syncthreads();
  constexpr int V = Vec<T>::N;
  for (int n = blockIdx.x * warps + warp; n < N; n += gridDim.x * warps) {
    const T* wr = W + ((size_t)h * N + n) * K;
    float acc[HV_ROWS];
#pragma unroll
    for (int r = 0; r < HV_ROWS; ++r) acc[r] = 0.f;
    if (K % V == 0 && (reinterpret_cast<uintptr_t>(wr) & 15) == 0) {
      for (int k = lane * V; k < K; k += 32 * V) {
        float f[V];
        unpack<T>(ldg_cached(wr + k), f);
#pragma unroll
        for (int r = 0; r < HV_ROWS; ++r)
          if (r < rows)
#pragma unroll
            for (int i = 0; i < V; ++i) acc[r] = fmaf(as[r * K + k + i], f[i], acc[r]);
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float f = to_f<T>(wr[k]);
#pragma unroll
        for (int r = 0; r < HV_ROWS; ++r)
          if (r < rows) acc[r] = fmaf(as[r * K + k], f, acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < HV_ROWS; ++r) {
      if (r >= rows) break;
      float v = warp_sum(acc[r]);
      if (lane == 0) {
        const int m = m0 + r;
        if (gate) v = rnd<T>(v) * (1.f / (1.f + expf(-to_f<T>(gate[(size_t)m * ldg + h * N + n]))));
        out[(size_t)m * ldo + h * o_hs + n] = from_f<T>(v);
      }
    }
  }
}

// out[m, h * o_hs + n] *= sigmoid(gate[m, h * N + n]), eight columns per thread: the gate of a per-head product that ran
// on the tensor cores (whose epilogue owns a row per thread and would read the gate 16 bytes at a time across 32 rows)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, int ldo, int o_hs, const T* __restrict__ gate, int ldg, unsigned M,
                                 unsigned heads, unsigned N) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = Vec<T>::N;
  const unsigned np = N / V, total = M * heads * np;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned n = (i % np) * V, r = i / np, h = r % heads, t = r / heads;
    T* o = out + (size_t)t * ldo + (size_t)h * o_hs + n;
    float f[V], g[V];
    unpack<T>(*reinterpret_cast<const uint4*>(o), f);
    unpack<T>(*reinterpret_cast<const uint4*>(gate + (size_t)t * ldg + h * N + n), g);
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] *= 1.f / (1.f + __expf(-g[j]));
    *reinterpret_cast<uint4*>(o) = pack<T>(f);
  }
}

// ------------------------------------------------------------------ [a | b] of two fp32 matrices in the model dtype
template <typename T>
__global__ void concat_cast_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                   long long rows, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = rows * 2 * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (2 * D);
    const int c = (int)(i % (2 * D));
    out[i] = from_f<T>(c < D ? a[r * D + c] : b[r * D + c - D]);
  }
}

bool head_gemm_tc_supported(int ldo, int o_gs, int lda, int a_gs, int N, int K, int dtype);
int head_gemm_tc(void* out, int ldo, int o_gs, const void* A, int lda, int a_gs, const void* W, int n_rows, int heads, int N,
                 int K, int dtype, int* err_flag, cudaStream_t st);

}  // namespace pg

using namespace pg;

extern "C" int pg_latent_prep(void* cq_out, const void* proj, int ld, int dq_col0, int q_rank, const void* w_q,
                              int dkv_col0, int kv_rank, const void* w_kv, int rot_dim, const float* freq, float mag,
                              float eps, void* pool, int ld_pool, const int32_t* page_table, int pt_stride,
                              int page_size, const int32_t* tok_slot, const int32_t* tok_pos, int n_tokens, int dtype,
                              void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(cq_out && proj && w_q && w_kv && pool && page_table && tok_slot && tok_pos && page_size > 0,
             "latent_prep: operands, pool and token map");
  PG_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && rot_dim % 2 == 0 && (rot_dim == 0 || freq) &&
                 ld_pool >= kv_rank + rot_dim,
             "latent_prep: ranks %d / %d, %d rotated columns, cache rows of %d", q_rank, kv_rank, rot_dim, ld_pool);
  PG_DISPATCH_DTYPE(dtype, T, {
    const int work = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = work >= 1024 ? 256 : 128;
    return launch_pdl("latent_prep", latent_prep_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream,
                      (T*)cq_out, (const T*)proj, ld, dq_col0, q_rank, (const T*)w_q, dkv_col0, kv_rank, (const T*)w_kv,
                      rot_dim, freq, mag, eps, (T*)pool, ld_pool, page_table, pt_stride, page_size, tok_slot, tok_pos);
  });
  return PG_OK;
}

extern "C" int pg_rotary_cols(void* dst, int ld_dst, int dst_col0, int dst_head_stride, const void* src, int ld_src,
                              int src_col0, int src_head_stride, int heads, int rot_dim, const float* freq, float mag,
                              const int32_t* tok_pos, int n_tokens, int dtype, void* stream) {
  if (n_tokens <= 0 || rot_dim <= 0) return PG_OK;
  PG_REQUIRE(dst && src && freq && tok_pos && rot_dim % 2 == 0 && heads > 0, "rotary_cols: bad arguments");
  PG_DISPATCH_DTYPE(dtype, T, {
    const int work = heads * rot_dim / 2;
    const int threads = work >= 512 ? 256 : (work >= 128 ? 128 : 64);
    return launch_pdl("rotary_cols", rotary_cols_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream,
                      (T*)dst, ld_dst, dst_col0, dst_head_stride, (const T*)src, ld_src, src_col0, src_head_stride, heads,
                      rot_dim, freq, mag, tok_pos);
  });
  return PG_OK;
}

extern "C" int pg_head_gemm_ex(void* out, int ldo, int out_head_stride, const void* A, int lda, int a_head_stride,
                               const void* W, const void* gate, int ld_gate, int n_rows, int heads, int N, int K, int impl,
                               int* err_flag, int dtype, void* stream) {
  if (n_rows <= 0) return PG_OK;
  PG_REQUIRE(out && A && W && heads > 0 && N > 0 && K > 0, "head_gemm: bad arguments");
  cudaStream_t st = (cudaStream_t)stream;
  // impl 0: prompt-sized 16-bit row counts on the tensor cores (all heads in one launch of the grouped kernel) where the
  // sizes allow; 1: the fp32-FMA kernels; 2: the tensor-core kernel or an error
  static const int tc_min_rows = env_int("PG_HEAD_GEMM_TC_MIN_ROWS", 64);
  const bool tc_ok = head_gemm_tc_supported(ldo, out_head_stride, lda, a_head_stride, N, K, dtype) &&
                     (long long)lda >= (long long)(heads - 1) * a_head_stride + K && (!gate || ld_gate % 8 == 0) &&
                     ((uintptr_t)gate % 16) == 0 && (long long)n_rows * heads * N < (1ll << 31);
  PG_REQUIRE(impl != 2 || tc_ok, "head_gemm: the tensor-core kernel does not take this problem (N=%d K=%d dtype %d)", N, K, dtype);
  if (impl == 2 || (impl == 0 && tc_ok && n_rows >= tc_min_rows)) {
    const int rc = head_gemm_tc(out, ldo, out_head_stride, A, lda, a_head_stride, W, n_rows, heads, N, K, dtype, err_flag, st);
    if (rc != PG_OK || !gate) return rc;
    const long long total = (long long)n_rows * heads * (N / 8);
    const int blocks = (int)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
    if (dtype == PG_BF16)
      return launch_pdl("head_gate", head_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, st, (bf16*)out, ldo, out_head_stride,
                        (const bf16*)gate, ld_gate, (unsigned)n_rows, (unsigned)heads, (unsigned)N);
    return launch_pdl("head_gate", head_gate_kernel<f16>, dim3(blocks), dim3(256), 0, st, (f16*)out, ldo, out_head_stride,
                      (const f16*)gate, ld_gate, (unsigned)n_rows, (unsigned)heads, (unsigned)N);
  }
  PG_DISPATCH_DTYPE(dtype, T, {
    if (n_rows <= 2 * HV_ROWS && (size_t)HV_ROWS * K * sizeof(float) <= 96 * 1024) {
      const int warps = 8;
      int col_ctas = cdiv(N, warps);
      if (col_ctas * heads > 1184) col_ctas = cdiv(1184, heads);       // about 8 CTAs per SM at most
      return launch_pdl("head_gemv", head_gemv_kernel<T>, dim3(col_ctas, heads, cdiv(n_rows, HV_ROWS)), dim3(warps * 32),
                        sizeof(float) * HV_ROWS * (size_t)K, st, (T*)out, ldo, out_head_stride, (const T*)A, lda,
                        a_head_stride, (const T*)W, (const T*)gate, ld_gate, n_rows, N, K);
    }
    return launch_pdl("head_gemm", head_gemm_kernel<T>, dim3(cdiv(N, HG_BN), cdiv(n_rows, HG_BM), heads), dim3(HG_THREADS),
                      0, st, (T*)out, ldo, out_head_stride, (const T*)A, lda, a_head_stride, (const T*)W, (const T*)gate,
                      ld_gate, n_rows, N, K);
  });
  return PG_OK;
}

extern "C" int pg_head_gemm(void* out, int ldo, int out_head_stride, const void* A, int lda, int a_head_stride,
                            const void* W, const void* gate, int ld_gate, int n_rows, int heads, int N, int K, int dtype,
                            void* stream) {
  return pg_head_gemm_ex(out, ldo, out_head_stride, A, lda, a_head_stride, W, gate, ld_gate, n_rows, heads, N, K, 1, nullptr,
                         dtype, stream);
}

extern "C" int pg_concat_cast(void* out, const float* a, const float* b, int rows, int D, int dtype, void* stream) {
  if (rows <= 0 || D <= 0) return PG_OK;
  PG_REQUIRE(out && a && b, "concat_cast: bad arguments");
  const long long n = (long long)rows * 2 * D;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("concat_cast", concat_cast_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out, a, b,
                      (long long)rows, D);
  });
  return PG_OK;
}
