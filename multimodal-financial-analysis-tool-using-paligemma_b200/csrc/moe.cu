// Mixture-of-experts feed-forward for token batches: router, grouping of the (token, expert) pairs by expert,
// grouped expert GEMMs and the weighted combination into the fp32 residual stream.
//
//   pg_moe_route    fp32 router logits, softmax over all routed outputs, top-k on (score + correction), weights =
//                   score * scale (not renormalised); optional per-token sigmoid gate of a shared expert
//   pg_moe_sort     pairs whose expert index is < n_experts are grouped by expert (offsets, source rows, position of
//                   each pair); larger indices are identity experts and take no part in the GEMMs
//   pg_moe_gemm     out[pos] = A[row(pos)] W_e^T for the pairs of every expert e, optionally with the SwiGLU pairing
//                   silu(A Wg^T) * (A Wu^T) of stacked [Wg; Wu] weights
//   pg_moe_combine  x[t] += sum_k w_k * (k-th expert's output, or the token's own input for an identity expert)
//                           + gate[t] * shared[t]
#include "common.cuh"

namespace pg {

// ------------------------------------------------------------------ router: one CTA per token
// The token's row sits in shared memory as fp32; warp w computes the logits of the routed outputs w, w + warps, ...
// (16-byte weight loads when the rows allow), then warp 0 does the softmax, the top-k and the weights.
template <typename T>
__device__ __forceinline__ float dot_smem(const float* __restrict__ hs, const T* __restrict__ wr, int D, int lane) {
  constexpr int V = Vec<T>::N;
  float acc = 0.f;
  if (D % V == 0 && (reinterpret_cast<uintptr_t>(wr) & 15) == 0) {
    for (int k = lane * V; k < D; k += 32 * V) {
      float f[V];
      unpack<T>(ldg_cached(wr + k), f);
#pragma unroll
      for (int i = 0; i < V; ++i) acc = fmaf(hs[k + i], f[i], acc);
    }
  } else {
    for (int k = lane; k < D; k += 32) acc = fmaf(hs[k], to_f<T>(wr[k]), acc);
  }
  return warp_sum(acc);
}

template <typename T>
__global__ void moe_route_kernel(int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                                 float* __restrict__ shared_gate, const T* __restrict__ h, int ldh,
                                 const T* __restrict__ w_router, const T* __restrict__ correction,
                                 const T* __restrict__ w_sg, int T_, int D, int n_route, int top, float scale) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  float* hs = smem;                               // [D]
  float* s = smem + D;                            // scores [n_route]
  float* c = s + n_route;                         // choice scores [n_route]
  const T* hr = h + (size_t)t * ldh;
  for (int k = threadIdx.x; k < D; k += blockDim.x) hs[k] = to_f<T>(hr[k]);
  __syncthreads();
  for (int e = warp; e < n_route + 1; e += warps) {
    if (e < n_route) {
      const float z = dot_smem<T>(hs, w_router + (size_t)e * D, D, lane);
      if (lane == 0) s[e] = z;
    } else if (w_sg && shared_gate) {
      const float z = dot_smem<T>(hs, w_sg, D, lane);
      if (lane == 0) shared_gate[t] = 1.f / (1.f + expf(-z));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float mx = -INFINITY;
  for (int e = lane; e < n_route; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < n_route; e += 32) sum += expf(s[e] - mx);
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < n_route; e += 32) {
    const float pr = expf(s[e] - mx) / sum;
    s[e] = pr;
    c[e] = pr + (correction ? to_f<T>(correction[e]) : 0.f);
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    unsigned long long best = 0ull;
    for (int e = lane; e < n_route; e += 32) {
      const unsigned long long key = argmax_key(c[e], (unsigned)e);
      best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = (int)argmax_key_index(best);
    if (lane == 0) {
      topk_idx[(size_t)t * top + k] = e;
      topk_w[(size_t)t * top + k] = s[e] * scale;
      c[e] = -INFINITY;
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------ router with sigmoid scores and expert groups: one CTA per token
// z = h W_router^T in fp32, s = sigmoid(z); the choice scores are c = s + correction.  The experts form n_groups equal
// groups of neighbours; a group's score is the sum of its two largest choice scores (of the one, for groups of one),
// and only the experts of the `keep` best groups can be chosen (the others' choice scores count as -inf).  The `top`
// largest choice scores are chosen (ties: lowest index); the weights are the chosen s (without the correction)
// divided by their sum + 1e-20.
template <typename T>
__global__ void moe_route_grouped_kernel(int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                                         const T* __restrict__ h, int ldh, const T* __restrict__ w_router,
                                         const T* __restrict__ correction, int T_, int D, int n_route, int top,
                                         int n_groups, int keep) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  float* hs = smem;                               // [D]
  float* s = smem + D;                            // scores [n_route]
  float* c = s + n_route;                         // choice scores [n_route]
  float* gs = c + n_route;                        // group scores [n_groups]
  const T* hr = h + (size_t)t * ldh;
  for (int k = threadIdx.x; k < D; k += blockDim.x) hs[k] = to_f<T>(hr[k]);
  __syncthreads();
  for (int e = warp; e < n_route; e += warps) {
    const float z = dot_smem<T>(hs, w_router + (size_t)e * D, D, lane);
    if (lane == 0) {
      const float sc = 1.f / (1.f + expf(-z));
      s[e] = sc;
      c[e] = sc + (correction ? to_f<T>(correction[e]) : 0.f);
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (n_groups > 1 && keep < n_groups) {
    const int gsz = n_route / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest of the group
      for (int e = g * gsz; e < (g + 1) * gsz; ++e) {
        const float v = c[e];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs[g] = gsz > 1 ? a + b : a;
    }
    __syncwarp();
    // the `keep` best groups are marked +inf one after the other; the groups left unmarked lose their experts
    for (int k = 0; k < keep; ++k) {
      unsigned long long best = 0ull;
      for (int g = lane; g < n_groups; g += 32) {
        if (gs[g] == INFINITY) continue;
        const unsigned long long key = argmax_key(gs[g], (unsigned)g);
        best = key > best ? key : best;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
      }
      if (lane == 0) gs[argmax_key_index(best)] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_route; e += 32)
      if (gs[e / gsz] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  for (int k = 0; k < top; ++k) {
    unsigned long long best = 0ull;
    for (int e = lane; e < n_route; e += 32) {
      if (s[e] < 0.f) continue;                    // chosen already (scores are sigmoids: never negative otherwise)
      const unsigned long long key = argmax_key(c[e], (unsigned)e);
      best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = (int)argmax_key_index(best);
    const float se = s[e];
    wsum += se;
    __syncwarp();
    if (lane == 0) {
      topk_idx[(size_t)t * top + k] = e;
      topk_w[(size_t)t * top + k] = se;
      s[e] = -1.f;
    }
    __syncwarp();
  }
  const float inv = 1.f / (wsum + 1e-20f);
  for (int k = lane; k < top; k += 32) topk_w[(size_t)t * top + k] *= inv;
}

// ------------------------------------------------------------------ group the pairs by expert (one CTA)
__global__ void moe_sort_kernel(int32_t* __restrict__ offsets, int32_t* __restrict__ sorted_row,
                                int32_t* __restrict__ pair_pos, const int32_t* __restrict__ topk_idx, int n_pairs,
                                int top, int n_experts) {
  extern __shared__ int sm_i[];
  pdl_launch_dependents();
  pdl_wait();
  int* count = sm_i;                   // [n_experts]
  int* cursor = sm_i + n_experts;      // [n_experts]
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < n_experts; ++e) { offsets[e] = acc; cursor[e] = acc; acc += count[e]; }
    offsets[n_experts] = acc;
  }
  __syncthreads();
  // the order of the pairs inside a group does not change any result: every output row is computed on its own
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < n_experts) {
      const int pos = atomicAdd(&cursor[e], 1);
      sorted_row[pos] = i / top;
      pair_pos[i] = pos;
    } else {
      pair_pos[i] = -1;
    }
  }
}

// ------------------------------------------------------------------ grouped GEMM, fp32 FMA (any dtype)
// The gated pairings of a stacked [Wg; Wu] product (g, u already rounded to the model dtype):
//   PG_GLU_SILU    silu(g) * u
//   PG_GLU_CLAMPED g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1)
template <typename T>
__device__ __forceinline__ float glu_pair(float g, float u, int act, float limit) {
  if (act == PG_GLU_CLAMPED) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return rnd<T>(g / (1.f + expf(-1.702f * g))) * (u + 1.f);
  }
  return rnd<T>(rnd<T>(g / (1.f + expf(-g))) * u);
}

constexpr int MG_BM = 64, MG_BN = 64, MG_BK = 16, MG_THREADS = 256, MG_PAD = 4;

template <typename T, bool DUAL>
__global__ void __launch_bounds__(MG_THREADS)
moe_gemm_simt_kernel(T* __restrict__ out, int ldo, const T* __restrict__ A, int lda,
                     const int32_t* __restrict__ row_map, const T* __restrict__ W,
                     const int32_t* __restrict__ offsets, int n_experts, int N, int K, int act, float limit) {
  __shared__ __align__(16) float As[MG_BK][MG_BM + MG_PAD];
  __shared__ __align__(16) float Bs[MG_BK][MG_BN + MG_PAD];
  __shared__ __align__(16) float Us[DUAL ? MG_BK : 1][MG_BN + MG_PAD];
  __shared__ int s_tile[3];
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int tile = blockIdx.y, e = 0, acc = 0;
    for (; e < n_experts; ++e) {
      const int nt = (offsets[e + 1] - offsets[e] + MG_BM - 1) / MG_BM;
      if (tile < acc + nt) break;
      acc += nt;
    }
    s_tile[0] = e;
    s_tile[1] = e < n_experts ? offsets[e] + (tile - acc) * MG_BM : 0;
    s_tile[2] = e < n_experts ? offsets[e + 1] : 0;
  }
  __syncthreads();
  const int e = s_tile[0], m0 = s_tile[1], m_end = s_tile[2];
  if (e >= n_experts) return;
  const int n0 = blockIdx.x * MG_BN;
  const int n_w = DUAL ? 2 * N : N;
  const T* We = W + (size_t)e * n_w * K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4], acu[DUAL ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (DUAL) acu[i][j] = 0.f; }
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    for (int idx = threadIdx.x; idx < MG_BM * MG_BK; idx += MG_THREADS) {
      const int r = idx / MG_BK, kk = idx % MG_BK;
      float a = 0.f, b = 0.f, u = 0.f;
      if (k0 + kk < K) {
        if (m0 + r < m_end) {
          const int src = row_map ? row_map[m0 + r] : m0 + r;
          a = to_f<T>(A[(size_t)src * lda + k0 + kk]);
        }
        if (n0 + r < N) {
          b = to_f<T>(We[(size_t)(n0 + r) * K + k0 + kk]);
          if (DUAL) u = to_f<T>(We[(size_t)(N + n0 + r) * K + k0 + kk]);
        }
      }
      As[kk][r] = a;
      Bs[kk][r] = b;
      if (DUAL) Us[kk][r] = u;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MG_BK; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      if (DUAL) {
        const float4 u = *reinterpret_cast<const float4*>(&Us[kk][tx * 4]);
        const float uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acu[i][j] = fmaf(av[i], uv[j], acu[i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = rnd<T>(acc[i][j]);
      if (DUAL) v = glu_pair<T>(v, rnd<T>(acu[DUAL ? i : 0][j]), act, limit);
      out[(size_t)m * ldo + n] = from_f<T>(v);
    }
  }
}

// ------------------------------------------------------------------ weighted combination into the residual stream
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ x, T* __restrict__ out, int ldo, const T* __restrict__ y, int ldy,
                                   const int32_t* __restrict__ pair_pos, const float* __restrict__ topk_w,
                                   const T* __restrict__ h, int ldh, const T* __restrict__ shared_out, int lds,
                                   const float* __restrict__ shared_gate, int D, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[(size_t)t * top + k];
      const float w = topk_w[(size_t)t * top + k];
      const float v = pos >= 0 ? to_f<T>(y[(size_t)pos * ldy + c]) : to_f<T>(h[(size_t)t * ldh + c]);
      acc = fmaf(w, v, acc);
    }
    if (shared_out) acc = fmaf(shared_gate ? shared_gate[t] : 1.f, to_f<T>(shared_out[(size_t)t * lds + c]), acc);
    if (out) out[(size_t)t * ldo + c] = from_f<T>(acc);
    else x[(size_t)t * D + c] += acc;
  }
}

// rows of the grouped order: out[pos] = a[row_map[pos]] (16-byte copies when the rows allow, else elements)
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ a, int lda,
                                   const int32_t* __restrict__ row_map, const int32_t* __restrict__ n_rows, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  if (n_rows && r >= *n_rows) return;
  const T* src = a + (size_t)row_map[r] * lda;
  T* dst = out + (size_t)r * cols;
  constexpr int V = Vec<T>::N;
  if (cols % V == 0 && lda % V == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = src[c];
  }
}

int moe_gemm_tc(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int act, float limit, int dtype,
                int* err_flag, cudaStream_t st);
bool moe_gemm_tc_supported(int ldo, int lda, const int32_t* row_map, int N, int K, int dtype);

}  // namespace pg

using namespace pg;

extern "C" int pg_moe_route(int32_t* topk_idx, float* topk_w, float* shared_gate, const void* h, int ldh,
                            const void* w_router, const void* correction, const void* w_shared_gate, int n_tokens,
                            int D, int n_route, int top, float scale, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(top >= 1 && top <= n_route && n_route <= 4096, "moe_route: top %d of %d routed outputs", top, n_route);
  const int warps = n_route + 1 < 8 ? 4 : 8;
  const size_t smem = sizeof(float) * ((size_t)D + 2 * (size_t)n_route);
  PG_REQUIRE(smem <= 200 * 1024, "moe_route: D=%d with %d routed outputs does not fit shared memory", D, n_route);
  PG_DISPATCH_DTYPE(dtype, T, {
    auto kern = moe_route_kernel<T>;
    return launch_pdl("moe_route", kern, dim3(n_tokens), dim3(warps * 32), smem, (cudaStream_t)stream, topk_idx, topk_w,
                      shared_gate, (const T*)h, ldh, (const T*)w_router, (const T*)correction, (const T*)w_shared_gate,
                      n_tokens, D, n_route, top, scale);
  });
  return PG_OK;
}

extern "C" int pg_moe_sort(int32_t* offsets, int32_t* sorted_row, int32_t* pair_pos, const int32_t* topk_idx,
                           int n_pairs, int top, int n_experts, void* stream) {
  PG_REQUIRE(n_experts >= 1 && n_experts <= 4096 && top >= 1, "moe_sort: %d experts, top %d", n_experts, top);
  return launch_pdl("moe_sort", moe_sort_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * (size_t)n_experts,
                    (cudaStream_t)stream, offsets, sorted_row, pair_pos, topk_idx, n_pairs, top, n_experts);
}

extern "C" int pg_moe_gemm_act(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                               const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int act, float limit,
                               int impl, int* err_flag, int dtype, void* stream) {
  if (n_pairs <= 0) return PG_OK;
  PG_REQUIRE(act == PG_GLU_NONE || act == PG_GLU_SILU || act == PG_GLU_CLAMPED, "moe_gemm: unknown pairing %d", act);
  const int swiglu = act != PG_GLU_NONE;
  cudaStream_t st = (cudaStream_t)stream;
  if (impl != 1 && moe_gemm_tc_supported(ldo, lda, row_map, N, K, dtype))
    return moe_gemm_tc(out, ldo, A, lda, row_map, W, offsets, n_pairs, n_experts, N, K, act, limit, dtype, err_flag, st);
  PG_REQUIRE(impl != 2, "moe_gemm: the tensor-core kernel does not take this problem (N=%d K=%d dtype %d)", N, K, dtype);
  dim3 grid(cdiv(N, MG_BN), cdiv(n_pairs, MG_BM) + n_experts);
  PG_DISPATCH_DTYPE(dtype, T, {
    if (swiglu)
      return launch_pdl("moe_gemm", moe_gemm_simt_kernel<T, true>, grid, dim3(MG_THREADS), 0, st, (T*)out, ldo, (const T*)A,
                        lda, row_map, (const T*)W, offsets, n_experts, N, K, act, limit);
    return launch_pdl("moe_gemm", moe_gemm_simt_kernel<T, false>, grid, dim3(MG_THREADS), 0, st, (T*)out, ldo, (const T*)A,
                      lda, row_map, (const T*)W, offsets, n_experts, N, K, act, limit);
  });
  return PG_OK;
}

extern "C" int pg_moe_gemm(void* out, int ldo, const void* A, int lda, const int32_t* row_map, const void* W,
                           const int32_t* offsets, int n_pairs, int n_experts, int N, int K, int swiglu, int impl,
                           int* err_flag, int dtype, void* stream) {
  return pg_moe_gemm_act(out, ldo, A, lda, row_map, W, offsets, n_pairs, n_experts, N, K,
                         swiglu ? PG_GLU_SILU : PG_GLU_NONE, 0.f, impl, err_flag, dtype, stream);
}

extern "C" int pg_moe_route_grouped(int32_t* topk_idx, float* topk_w, const void* h, int ldh, const void* w_router,
                                    const void* correction, int n_tokens, int D, int n_route, int top, int n_groups,
                                    int keep, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(top >= 1 && top <= n_route && n_route <= 4096, "moe_route: top %d of %d routed outputs", top, n_route);
  PG_REQUIRE(n_groups >= 1 && n_route % n_groups == 0 && keep >= 1 && keep <= n_groups &&
                 (long long)keep * (n_route / n_groups) >= top,
             "moe_route: %d groups over %d experts, %d kept, top %d", n_groups, n_route, keep, top);
  const int warps = n_route < 8 ? 4 : 8;
  const size_t smem = sizeof(float) * ((size_t)D + 2 * (size_t)n_route + n_groups);
  PG_REQUIRE(smem <= 200 * 1024, "moe_route: D=%d with %d routed outputs does not fit shared memory", D, n_route);
  PG_DISPATCH_DTYPE(dtype, T, {
    auto kern = moe_route_grouped_kernel<T>;
    return launch_pdl("moe_route_grouped", kern, dim3(n_tokens), dim3(warps * 32), smem, (cudaStream_t)stream, topk_idx,
                      topk_w, (const T*)h, ldh, (const T*)w_router, (const T*)correction, n_tokens, D, n_route, top,
                      n_groups, keep);
  });
  return PG_OK;
}

static int moe_combine_any(float* x, void* out, int ldo, const void* y, int ldy, const int32_t* pair_pos,
                           const float* topk_w, const void* h, int ldh, const void* shared_out, int lds,
                           const float* shared_gate, int n_tokens, int D, int top, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_DISPATCH_DTYPE(dtype, T, {
    const int threads = n_tokens <= 64 ? (D >= 2048 ? 512 : 256) : 128;
    return launch_pdl("moe_combine", moe_combine_kernel<T>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, x,
                      (T*)out, ldo, (const T*)y, ldy, pair_pos, topk_w, (const T*)h, ldh, (const T*)shared_out, lds,
                      shared_gate, D, top);
  });
  return PG_OK;
}

extern "C" int pg_moe_combine(float* x, const void* y, int ldy, const int32_t* pair_pos, const float* topk_w,
                              const void* h, int ldh, const void* shared_out, int lds, const float* shared_gate,
                              int n_tokens, int D, int top, int dtype, void* stream) {
  return moe_combine_any(x, nullptr, 0, y, ldy, pair_pos, topk_w, h, ldh, shared_out, lds, shared_gate, n_tokens, D, top,
                         dtype, stream);
}

extern "C" int pg_moe_combine_out(void* out, int ldo, const void* y, int ldy, const int32_t* pair_pos,
                                  const float* topk_w, const void* shared_out, int lds, int n_tokens, int D, int top,
                                  int dtype, void* stream) {
  PG_REQUIRE(out && ldo >= D, "moe_combine_out: an output of %d columns", D);
  return moe_combine_any(nullptr, out, ldo, y, ldy, pair_pos, topk_w, nullptr, 0, shared_out, lds, nullptr, n_tokens, D,
                         top, dtype, stream);
}

extern "C" int pg_gather_rows(void* out, const void* a, int lda, const int32_t* row_map, const int32_t* n_rows,
                              int max_rows, int cols, int dtype, void* stream) {
  if (max_rows <= 0) return PG_OK;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("gather_rows", gather_rows_kernel<T>, dim3(max_rows), dim3(128), 0, (cudaStream_t)stream, (T*)out,
                      (const T*)a, lda, row_map, n_rows, cols);
  });
  return PG_OK;
}
