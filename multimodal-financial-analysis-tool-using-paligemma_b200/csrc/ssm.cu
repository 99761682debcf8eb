// Selective state-space mixer (the scalar-decay form: one decay per head and token) for ragged token batches.
//
// The fused input projection of a token holds [z: inner | x: inner | B: G N | C: G N | dt: H] (inner = H vdim, H heads,
// G groups of heads that share B and C, N the state size).  x, B and C pass a causal convolution over time per channel
// (taps columns, the last one the current token's, plus a bias) and silu; step = softplus(dt + dt_bias) (no clamp);
// per head, with the state S [N x vdim] kept in fp32 per sequence slot:
//     S <- exp(-exp(A_log_h) step) S + step B x^T,      y = S^T C + D_h x.
// This is the recurrence of the decayed linear-attention kernel (recurrent.cu) with key step * B, value x, query C, a
// decay per (token, head) and a skip term; ssm_prep_kernel writes exactly its records and that kernel runs the scan.
//
// ssm_prep_kernel       (CTA per token; every channel is convolved once into shared memory, then the records of all
//                       heads are written from there): the convolution reads the token's own row and the taps - 1 inputs before it,
//                       rows of the same step where the sequence has them, else the slot's convolution state
//                       (timeconv.cu keeps it: the last taps - 1 projected inputs, fp32); conv, silu, softplus and
//                       both exponentials in fp32.  One packed fp32 record per (token, head):
//                       [C (np) | step * B (np) | x (vp) | decay, 0, 0, 0], np / vp = N / vdim rounded up to 4 floats.
// gate_groupnorm_kernel (warp per (token, norm group)): y * silu(z) first, then each of the `groups` equal parts of the
//                       row is divided by its own root mean square and multiplied by the weight; fp32, one rounding to
//                       the model dtype (the output projection's operand).
#include "common.cuh"

namespace pg {

__device__ __forceinline__ float ssm_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float ssm_silu(float v) { return v / (1.f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(256)
ssm_prep_kernel(float* __restrict__ rec, const T* __restrict__ proj, int ld, int xbc_col0, int dt_col0,
                const T* __restrict__ conv_w, const T* __restrict__ conv_b, const float* __restrict__ conv_state,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const int32_t* __restrict__ tok_slot,
                int heads, int vdim, int N, int groups, int taps, int np, int vp) {
  extern __shared__ float sm[];                    // [heads] step | [heads] decay | [channels] silu(conv) of x, B, C
  float* step = sm;
  float* decay = sm + heads;
  float* act = sm + 2 * heads;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, K = taps - 1, inner = heads * vdim, channels = inner + 2 * groups * N;
  const int slot = tok_slot[t];
  int before = 0;                                  // rows of the same sequence right before this one, up to K
  while (before < K && t - before - 1 >= 0 && tok_slot[t - before - 1] == slot) ++before;
  const T* row = proj + (size_t)t * ld;
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float s = ssm_softplus(to_f<T>(row[dt_col0 + h]) + dt_bias[h]);
    step[h] = s;
    decay[h] = expf(-expf(a_log[h]) * s);
  }
  // every channel once (B and C are shared by the heads of a group): consecutive threads, consecutive channels
  for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) {
    const T* wc = conv_w + (size_t)ch * taps;
    float acc = to_f<T>(conv_b[ch]);
    acc = fmaf(to_f<T>(row[xbc_col0 + ch]), to_f<T>(wc[K]), acc);
    for (int j = 1; j <= K; ++j) {
      const float u = j <= before ? to_f<T>(proj[(size_t)(t - j) * ld + xbc_col0 + ch])
                                  : conv_state[((size_t)slot * K + (K - (j - before))) * channels + ch];
      acc = fmaf(u, to_f<T>(wc[K - j]), acc);
    }
    act[ch] = ssm_silu(acc);
  }
  __syncthreads();
  // a warp per head writes its record in four floats per lane (np and vp are multiples of 4, so a vector never
  // straddles two parts of the record)
  const int rs = 2 * np + vp + 4, hpg = heads / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < heads; h += blockDim.x >> 5) {
    const int g = h / hpg;
    const float* cq = act + inner + groups * N + g * N;      // C: the query
    const float* bk = act + inner + g * N;                   // B: the key, times the step
    const float* xv = act + h * vdim;                        // x: the value
    const float sh = step[h];
    float* out = rec + ((size_t)t * heads + h) * rs;
    for (int c = lane * 4; c < rs; c += 128) {
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int cc = c + i;
        float a = 0.f;
        if (cc < np) { if (cc < N) a = cq[cc]; }
        else if (cc < 2 * np) { if (cc - np < N) a = bk[cc - np] * sh; }
        else if (cc < 2 * np + vp) { if (cc - 2 * np < vdim) a = xv[cc - 2 * np]; }
        else if (cc == 2 * np + vp) a = decay[h];
        v[i] = a;
      }
      *reinterpret_cast<float4*>(out + c) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

template <typename T>
__global__ void gate_groupnorm_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ y, const T* __restrict__ z,
                                      int ld_z, const T* __restrict__ w, int n_tokens, int cols, int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_tokens * groups) return;
  const int t = item / groups, g = item % groups, gs = cols / groups;
  const float* yr = y + (size_t)t * cols + g * gs;
  const T* zr = z + (size_t)t * ld_z + g * gs;
  float ss = 0.f;
  for (int c = lane; c < gs; c += 32) { const float v = yr[c] * ssm_silu(to_f<T>(zr[c])); ss += v * v; }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)gs + eps);
  T* o = out + (size_t)t * ld_out + g * gs;
  for (int c = lane; c < gs; c += 32)
    o[c] = from_f<T>(yr[c] * ssm_silu(to_f<T>(zr[c])) * inv * (w ? to_f<T>(w[g * gs + c]) : 1.f));
}

}  // namespace pg

using namespace pg;

extern "C" long long pg_ssm_record_floats(int n_tokens, int heads, int vdim, int state) {
  return (long long)n_tokens * heads * (2 * ((state + 3) / 4 * 4) + (vdim + 3) / 4 * 4 + 4);
}

extern "C" int pg_ssm_prep(float* rec, const void* proj, int ld, int xbc_col0, int dt_col0, const void* conv_w,
                           const void* conv_b, const float* conv_state, const float* dt_bias, const float* a_log,
                           const int32_t* tok_slot, int n_tokens, int heads, int vdim, int state, int groups, int taps,
                           int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(rec && proj && conv_w && conv_b && dt_bias && a_log && tok_slot && (taps == 1 || conv_state),
             "ssm_prep: bad arguments");
  PG_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && taps >= 1, "ssm_prep: %d heads in %d groups, %d taps", heads,
             groups, taps);
  const int np = (state + 3) / 4 * 4, vp = (vdim + 3) / 4 * 4;
  PG_DISPATCH_DTYPE(dtype, T, {
    const size_t smem = sizeof(float) * (2 * (size_t)heads + (size_t)heads * vdim + 2 * (size_t)groups * state);
    return launch_pdl("ssm_prep", ssm_prep_kernel<T>, dim3(n_tokens), dim3(256), smem,
                      (cudaStream_t)stream, rec, (const T*)proj, ld, xbc_col0, dt_col0, (const T*)conv_w, (const T*)conv_b,
                      conv_state, dt_bias, a_log, tok_slot, heads, vdim, state, groups, taps, np, vp);
  });
  return PG_OK;
}

extern "C" int pg_gate_groupnorm(void* out, int ld_out, const float* y, const void* z, int ld_z, const void* w, int n_tokens,
                                 int cols, int groups, float eps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && y && z && groups >= 1 && cols % groups == 0, "gate_groupnorm: %d columns in %d groups", cols, groups);
  const int warps = 8;
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("gate_groupnorm", gate_groupnorm_kernel<T>, dim3(cdiv((long long)n_tokens * groups, warps)),
                      dim3(warps * 32), 0, (cudaStream_t)stream, (T*)out, ld_out, y, (const T*)z, ld_z, (const T*)w, n_tokens,
                      cols, groups, eps);
  });
  return PG_OK;
}
