// Short causal convolutions over time for ragged token batches, with the last inputs of every sequence kept as state.
//
// A convolution of `taps` taps over time on each channel reads, for the token at position p, the inputs of positions
// p - taps + 1 .. p of its sequence (zeros before the sequence's start).  In a step, the tokens of a sequence are
// consecutive rows at consecutive positions, so the input j positions back is row t - j when the sequence has that many
// rows before row t in this step, and otherwise comes from the sequence's state: the last taps - 1 inputs that earlier
// steps saw, fp32 [slots][taps - 1][channels], entry taps - 2 the most recent, all zero for a new sequence.  How many
// rows of its sequence precede a token is read off the token map (rows of one sequence carry the same slot).
//
// time_conv_residual_kernel : out = in + conv(in) on fp32 rows (the normalised residual stream), weights [C][taps]
//                             in the model dtype, the last column the current token's; fp32 sum, one rounding to the
//                             model dtype (the operand of the sublayer's projection).
// time_conv_state_kernel    : after the step's last reader of the state: per segment {slot, first row, tokens}, the
//                             state becomes the last taps - 1 entries of [old state ; the segment's inputs].  A
//                             thread owns a channel and writes the entries in ascending order, each from an older
//                             entry or from a row, so the update is in place.  Segments of 0 tokens are skipped.
//                             Its source is fp32 rows or model-dtype columns of a projection (the recurrent mixers'
//                             own convolutions keep their state the same way).
//
// norm_time_conv_kernel     : the residual sum, the RMS norm and the convolution of a sublayer's input in ONE pass.  A CTA
//                             owns TOK consecutive rows: x_out = x_in + y for them, and h = n + conv(n) with
//                             n = x_out / rms(x_out) * (w or 1 + w).  The normed rows of the K = taps - 1 rows before the
//                             tile are recomputed from x_in + y (their statistics cost K more row reads per tile, out of
//                             L2), which is why x_out must not alias x_in: the CTA that owns those rows writes them
//                             meanwhile.  A thread then walks the tile's rows of its channels with the last K normed
//                             values in registers, refilled from the sequence's state where a sequence starts inside
//                             the tile or the step.
// norm_time_conv_state_kernel: the state update for that kernel, which leaves no normed rows behind: the K rows a segment
//                             ends with are normed again from x_out (a CTA per segment and entry; a segment shorter
//                             than K also moves old entries down, in order, in one CTA).
#include "common.cuh"

namespace pg {

constexpr int CONV_MAX_TAPS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
time_conv_residual_kernel(T* __restrict__ out, const float* __restrict__ in, const T* __restrict__ w,
                          const float* __restrict__ state, const int32_t* __restrict__ tok_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, K = taps - 1;
  const int slot = tok_slot[t];
  int before = 0;                                  // rows of the same sequence right before this one, up to K
  while (before < K && t - before - 1 >= 0 && tok_slot[t - before - 1] == slot) ++before;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const T* wc = w + (size_t)c * taps;
    const float cur = in[(size_t)t * C + c];
    float acc = cur * to_f<T>(wc[K]);
    for (int j = 1; j <= K; ++j) {
      const float v = j <= before ? in[(size_t)(t - j) * C + c]
                                  : state[((size_t)slot * K + (K - (j - before))) * C + c];
      acc = fmaf(v, to_f<T>(wc[K - j]), acc);
    }
    out[(size_t)t * C + c] = from_f<T>(cur + acc);
  }
}

template <typename TS>
__global__ void __launch_bounds__(256)
time_conv_state_kernel(float* __restrict__ state, const TS* __restrict__ src, int ld, int col0,
                       const int32_t* __restrict__ segs, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2], K = taps - 1;
  if (n <= 0) return;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float* st = state + (size_t)slot * K * C + c;
    for (int i = 0; i < K; ++i) {                  // entry i of the new state = entry n + i of [old state ; rows]
      const int idx = n + i;
      st[(size_t)i * C] = idx < K ? st[(size_t)idx * C] : to_f<TS>(src[(size_t)(row0 + idx - K) * ld + col0 + c]);
    }
  }
}

// VEC consecutive channels of x (+ y): one 16-byte load of the stream and one of 4 model-dtype values, or single elements
template <typename T, int VEC>
__device__ __forceinline__ void load_sum(const float* __restrict__ x, const T* __restrict__ y, float* v) {
  if constexpr (VEC == 4) {
    const float4 a = *reinterpret_cast<const float4*>(x);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    if (y) {
      if constexpr (sizeof(T) == 4) {
        const float4 b = *reinterpret_cast<const float4*>(y);
        v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(y);
        const T* t = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += to_f<T>(t[i]);
      }
    }
  } else {
    v[0] = x[0] + (y ? to_f<T>(y[0]) : 0.f);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* __restrict__ dst, const float* v) {
  if constexpr (VEC == 4) {
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      uint2 u;
      T* t = reinterpret_cast<T*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) t[i] = from_f<T>(v[i]);
      *reinterpret_cast<uint2*>(dst) = u;
    }
  } else {
    dst[0] = from_f<T>(v[0]);
  }
}

template <typename T, int TOK, int VEC, int KM>     // KM: the most rows back this instance keeps in registers (taps - 1 <= KM)
__global__ void __launch_bounds__(256)
norm_time_conv_kernel(T* __restrict__ out, float* __restrict__ x_out, const float* __restrict__ x_in,
                      const T* __restrict__ y, int ldy, const T* __restrict__ w_norm, int one_plus, float eps,
                      const T* __restrict__ w_conv, const float* __restrict__ state, const int32_t* __restrict__ tok_slot,
                      int n_tokens, int D, int taps) {
  __shared__ float inv[TOK + KM];                  // 1 / rms of rows t0 - K .. t0 + TOK - 1
  __shared__ int bef[TOK], slot_of[TOK];
  pdl_launch_dependents();
  pdl_wait();
  const int K = taps - 1, t0 = blockIdx.x * TOK, nt = min(TOK, n_tokens - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (threadIdx.x < nt) {
    const int t = t0 + threadIdx.x, slot = tok_slot[t];
    int b = 0;
    while (b < K && t - b - 1 >= 0 && tok_slot[t - b - 1] == slot) ++b;
    bef[threadIdx.x] = b;
    slot_of[threadIdx.x] = slot;
  }
  for (int r = warp - K; r < nt; r += warps) {     // a warp per row: the sum (written for the tile's own rows) and its rms
    const int t = t0 + r;
    if (t < 0) continue;
    const float* xr = x_in + (size_t)t * D;
    const T* yr = y ? y + (size_t)t * ldy : nullptr;
    float ss = 0.f;
#pragma unroll 8
    for (int c = lane * VEC; c < D; c += 32 * VEC) {
      float v[VEC];
      load_sum<T, VEC>(xr + c, yr ? yr + c : nullptr, v);
      if (r >= 0) store_vec<float, VEC>(x_out + (size_t)t * D + c, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) ss += v[i] * v[i];
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[r + K] = 1.f / sqrtf(ss / (float)D + eps);
  }
  __syncthreads();
  const float w0 = one_plus ? 1.f : 0.f;
  for (int c = threadIdx.x * VEC; c < D; c += blockDim.x * VEC) {
    float wn[VEC], wr[KM + 1][VEC], prev[KM][VEC];   // wr[j]: the tap j rows back; prev[j - 1]: the normed value j rows back
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      wn[i] = w0 + to_f<T>(w_norm[c + i]);
#pragma unroll
      for (int j = 0; j <= KM; ++j) wr[j][i] = j <= K ? to_f<T>(w_conv[(size_t)(c + i) * taps + K - j]) : 0.f;
    }
    auto normed = [&](int r, float* v) {           // row t0 + r of these channels
      const size_t t = (size_t)(t0 + r);
      load_sum<T, VEC>(x_in + t * D + c, y ? y + t * ldy + c : nullptr, v);
      const float iv = inv[r + K];
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] *= iv * wn[i];
    };
#pragma unroll 4
    for (int r = 0; r < nt; ++r) {
      const int b = bef[r];
      if (r == 0 || b < K) {                       // the tile's first row, or a sequence that starts within K rows
#pragma unroll
        for (int j = 1; j <= KM; ++j)
          if (j <= K) {
            if (j <= b) { if (r == 0) normed(-j, prev[j - 1]); }
            else {
              const float* sp = state + ((size_t)slot_of[r] * K + (K - (j - b))) * D + c;
#pragma unroll
              for (int i = 0; i < VEC; ++i) prev[j - 1][i] = sp[i];
            }
          }
      }
      float cur[VEC], o[VEC];
      normed(r, cur);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float acc = cur[i] * wr[0][i];
#pragma unroll
        for (int j = 1; j <= KM; ++j)
          if (j <= K) acc = fmaf(prev[j - 1][i], wr[j][i], acc);
        o[i] = cur[i] + acc;
      }
      store_vec<T, VEC>(out + (size_t)(t0 + r) * D + c, o);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
#pragma unroll
        for (int j = KM; j >= 2; --j)
          if (j <= K) prev[j - 1][i] = prev[j - 2][i];
        if (K >= 1) prev[0][i] = cur[i];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
norm_time_conv_state_kernel(float* __restrict__ state, const float* __restrict__ x, const T* __restrict__ w_norm,
                            int one_plus, float eps, const int32_t* __restrict__ segs, int D, int taps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int32_t* sg = segs + 3 * (size_t)blockIdx.x;
  const int slot = sg[0], row0 = sg[1], n = sg[2], K = taps - 1;
  if (n <= 0) return;
  const float w0 = one_plus ? 1.f : 0.f;
  float* st = state + (size_t)slot * K * D;
  // a segment of K rows or more fills every entry from a row: one CTA per entry (blockIdx.y).  A shorter one also
  // moves old entries down, in order: the first CTA does it all.
  const bool split = n >= K;
  if (!split && blockIdx.y != 0) return;
  for (int i = split ? blockIdx.y : 0; i < (split ? blockIdx.y + 1 : K); ++i) {   // entry i of the new state = entry n + i of [old state ; normed rows]
    const int idx = n + i;
    if (idx < K) {
      for (int c = threadIdx.x; c < D; c += blockDim.x) st[(size_t)i * D + c] = st[(size_t)idx * D + c];
      continue;
    }
    const float* xr = x + (size_t)(row0 + idx - K) * D;
    float ss = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) ss += xr[c] * xr[c];
    ss = block_sum(ss, red);
    const float iv = 1.f / sqrtf(ss / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) st[(size_t)i * D + c] = xr[c] * iv * (w0 + to_f<T>(w_norm[c]));
  }
}

}  // namespace pg

using namespace pg;

extern "C" int pg_norm_time_conv(void* out, float* x_out, const float* x_in, const void* y, int ldy, const void* w_norm,
                                 int one_plus, float eps, const void* w_conv, float* state, const int32_t* tok_slot,
                                 const int32_t* segs, int n_segs, int n_tokens, int D, int taps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && x_out && x_in && x_out != x_in && w_norm && w_conv && tok_slot && D > 0, "norm_time_conv: bad arguments");
  PG_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS && (taps == 1 || (state && segs)), "norm_time_conv: %d taps (1..%d)", taps,
             CONV_MAX_TAPS);
  cudaStream_t st = (cudaStream_t)stream;
  // rows per CTA: a tile re-reads the taps - 1 rows before it, so long tiles for prompt portions; a row per CTA for a
  // handful of tokens (decode steps), where the launch must spread over the SMs.  Four channels per thread where the
  // rows allow 16-byte accesses.
  int tok = n_tokens <= 64 ? 1 : (n_tokens <= 1024 ? 4 : 16);
  PG_DISPATCH_DTYPE(dtype, T, {
    const bool vec = D % 4 == 0 && (!y || (ldy % 4 == 0 && ((uintptr_t)y % 16) == 0)) && ((uintptr_t)x_in % 16) == 0 &&
                     ((uintptr_t)x_out % 16) == 0 && ((uintptr_t)out % 16) == 0 && (!state || ((uintptr_t)state % 16) == 0);
    constexpr int KL = CONV_MAX_TAPS - 1;           // up to 4 taps keep 3 rows back in registers (twice the CTAs per SM)
    auto kern = tok == 1 ? (vec ? norm_time_conv_kernel<T, 1, 4, KL> : norm_time_conv_kernel<T, 1, 1, KL>)
                         : (tok == 4 ? (vec ? norm_time_conv_kernel<T, 4, 4, KL> : norm_time_conv_kernel<T, 4, 1, KL>)
                                     : (vec ? norm_time_conv_kernel<T, 16, 4, KL> : norm_time_conv_kernel<T, 16, 1, KL>));
    if (taps <= 4)
      kern = tok == 1 ? (vec ? norm_time_conv_kernel<T, 1, 4, 3> : norm_time_conv_kernel<T, 1, 1, 3>)
                      : (tok == 4 ? (vec ? norm_time_conv_kernel<T, 4, 4, 3> : norm_time_conv_kernel<T, 4, 1, 3>)
                                  : (vec ? norm_time_conv_kernel<T, 13, 4, 3> : norm_time_conv_kernel<T, 13, 1, 3>));
    if (taps <= 4 && tok == 16) tok = 13;            // 13 + 3 rows of statistics: two full rounds of the CTA's 8 warps
    int rc = launch_pdl("norm_time_conv", kern, dim3(cdiv(n_tokens, tok)), dim3(256), 0, st, (T*)out,
                        x_out, x_in, (const T*)y, ldy, (const T*)w_norm, one_plus, eps, (const T*)w_conv, (const float*)state,
                        tok_slot, n_tokens, D, taps);
    if (rc != PG_OK || taps == 1 || n_segs <= 0) return rc;
    return launch_pdl("norm_time_conv_state", norm_time_conv_state_kernel<T>, dim3(n_segs, taps - 1), dim3(256), 0, st, state,
                      (const float*)x_out, (const T*)w_norm, one_plus, eps, segs, D, taps);
  });
  return PG_OK;
}

extern "C" int pg_time_conv_residual(void* out, const float* in, const void* w, const float* state,
                                     const int32_t* tok_slot, int n_tokens, int C, int taps, int dtype, void* stream) {
  if (n_tokens <= 0) return PG_OK;
  PG_REQUIRE(out && in && w && tok_slot && C > 0 && taps >= 1 && (taps == 1 || state), "time_conv_residual: bad arguments");
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("time_conv_residual", time_conv_residual_kernel<T>, dim3(n_tokens, cdiv(C, 1024)), dim3(256), 0,
                      (cudaStream_t)stream, (T*)out, in, (const T*)w, state, tok_slot, C, taps);
  });
  return PG_OK;
}

extern "C" int pg_time_conv_state(float* state, const void* src, int ld, int col0, int src_f32, const int32_t* segs,
                                  int n_segs, int C, int taps, int dtype, void* stream) {
  if (n_segs <= 0 || taps <= 1) return PG_OK;
  PG_REQUIRE(state && src && segs && C > 0 && ld >= C, "time_conv_state: bad arguments");
  const dim3 grid(n_segs, cdiv(C, 256));
  if (src_f32)
    return launch_pdl("time_conv_state", time_conv_state_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, state,
                      (const float*)src, ld, col0, segs, C, taps);
  PG_DISPATCH_DTYPE(dtype, T, {
    return launch_pdl("time_conv_state", time_conv_state_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, state,
                      (const T*)src, ld, col0, segs, C, taps);
  });
  return PG_OK;
}
